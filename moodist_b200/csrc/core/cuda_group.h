// CUDA side of a process group: owns the group's symmetric memory, the collective sequence number and
// the stream-ordering event, picks a kernel variant per call and launches it.
//
// All collectives are stream-ordered on the caller's stream and return immediately, like the
// reference's CUDA paths (wrapper/processgroup_wrapper.cc:63-85 hands back an already-complete Work).
// Collectives of one group are serialised with an event so they reach the GPUs in the same order on
// every rank even when issued from different streams (the reference uses a 16-slot ring of events,
// core/processgroup.cc:121-130, 318, 1111).
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <map>
#include <string>
#include <vector>

#include "kvstore.h"

struct CUstream_st;

namespace moodist {

struct GroupOptions {
  // names follow the reference's per-group options (core/processgroup.cc:334-340)
  int prefer_kernel_less = 0;
  int force_kernel_less = 0;
  int num_chunks = -1;
  int chunk_size = -1;
  int method = -1;  // -1 auto, 0 P2P kernels, 1 NVLS kernels, 2 copy engine (DMA copies between flag kernels)
};

// One row of CudaGroup::stats(): an operation and the kernel family that served it ("all_gather/nvls").
struct OpStat {
  std::string name;
  uint64_t calls = 0;
  uint64_t bytes = 0;        // payload bytes of all calls
  uint64_t timed_calls = 0;  // calls whose device time was sampled (every MOODIST_STATS_SAMPLE-th, default 64)
  double device_us = 0;      // summed device time of the sampled calls
};

// Thresholds for `world` ranks from a MOODIST_VARIANT_TABLE file ({"<world>": {"MOODIST_...": integer}});
// empty when the file is missing or malformed (an error is logged and the built-in values stay).
std::map<std::string, long> load_variant_table(const std::string& path, int world);

class CudaGroup {
 public:
  static std::unique_ptr<CudaGroup> create(KVStore& store, const std::string& key, int rank, int world, int device);
  virtual ~CudaGroup() = default;

  virtual int rank() const = 0;
  virtual int world() const = 0;
  virtual int device() const = 0;
  virtual bool has_nvls() const = 0;
  virtual int numa_node() const = 0;  // memory node of this rank's GPU, -1 when unknown
  virtual GroupOptions& options() = 0;

  virtual void all_gather(const void* in, void* out, size_t count, int in_dtype, int out_dtype, CUstream_st* s) = 0;
  virtual void reduce_scatter(const void* in, void* out, size_t count, int in_dtype, int out_dtype, int op,
                              float premul, CUstream_st* s) = 0;
  virtual void all_reduce(const void* in, void* out, size_t count, int dtype, int op, float premul,
                          CUstream_st* s) = 0;
  virtual void broadcast(void* data, size_t bytes, int root, CUstream_st* s) = 0;
  // byte offsets / counts per peer, arrays of length world
  virtual void all_to_all(const void* in, void* out, const uint64_t* send_off, const uint64_t* send_bytes,
                          const uint64_t* recv_off, const uint64_t* recv_bytes, CUstream_st* s) = 0;
  virtual void barrier(CUstream_st* s) = 0;

  // Raw access for fused ops and compile_op lowering.
  virtual const void* comm_struct() const = 0;          // mb_comm_t*
  virtual uint32_t next_seq(CUstream_st* s) = 0;        // orders the caller's launch after earlier ops
  virtual void finish_op(CUstream_st* s) = 0;           // records the ordering event after the launch
  virtual void* scratch(size_t bytes) = 0;              // small device buffer for tables (grown on demand)

  // Throws moodist::Error if a device-side wait ran out since the last check.
  virtual void check_status() = 0;
  virtual uint64_t launches() const = 0;                // kernels launched by this group so far
  // Per-op counters (the reference keeps byte counters per group, core/group.h:217-232). wait: block until the
  // sampled event pairs still in flight have finished.
  virtual std::vector<OpStat> stats(bool wait) = 0;
  virtual void note_op(const char* op, const char* variant, size_t bytes) = 0;  // for ops launched by the glue
  virtual std::string describe() const = 0;
};

}  // namespace moodist
