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
#include <string>

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

struct OpCounters {
  uint64_t calls = 0;
  uint64_t bytes = 0;
  uint64_t launches = 0;
};

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
  virtual std::string describe() const = 0;
};

}  // namespace moodist
