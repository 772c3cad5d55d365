// Host side of a process group: the progress engine ("moodist-cputhread") that owns the TCP data
// plane, runs CPU-tensor collectives, the Queue protocol, compile_op execution across hosts, the
// heartbeat and the coordinated shutdown. Needs no GPU and no CUDA library.
//
// Reference: core/cputhread.cc (engine + coroutine-style Work objects, :1080-1138, :6101-6340),
// core/rdma_tcp.cc + core/tcpdev.cc (TCP emulation of one-sided RDMA), core/setup_comms.cc (bootstrap).
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "kvstore.h"
#include "wire.h"

namespace moodist {

// Engine message types. The numeric values are the ones the reference puts on the wire (they are the
// source line numbers of its enum, core/cputhread.h:60-98), spelled out here as constants.
enum OpType : uint32_t {
  kOpBarrier = 60,
  kOpInternalBarrier = 61,
  kOpAllGatherCpu = 62,
  kOpReduceScatterCpu = 63,
  kOpBroadcastRingCpu = 64,
  kOpGatherCpu = 65,
  kOpAllToAllCpu = 66,  // not in the reference (its all_to_all is CUDA-only)
  kOpAllGatherKernelLessCuda = 67,
  kOpAllGatherLocalCuda = 68,
  kOpReduceScatterKernelLessCuda = 72,
  kOpBroadcastCuda = 75,
  kOpReduceCuda = 76,
  kOpAllToAllCuda = 77,
  kOpBarrierCuda = 81,
  kOpCreateQueue = 86,
  kOpQueuePut = 87,
  kOpQueueReadFinished = 88,
  kOpQueueGet = 89,
  kOpQueueTransaction = 90,
  kOpCreateQueueNamed = 91,
  kOpCreateQueueNamedResult = 92,
  kOpCustom = 96,
  kOpMessageShutdown = 98,
  kOpHeartbeat = 99,    // the reference heartbeats with RDMA writes; over plain TCP it is a message
  kOpScatterCpu = 100,  // not in the reference (scatter throws there)
  kOpSendRecv = 101,    // point-to-point payloads (send/recv are unsupported in the reference)
  kOpCudaItemDone = 103, // a receiver has copied a point-to-point CUDA tensor: the sender may release its buffer
  kOpSendOffer = 104,    // a large point-to-point payload is ready to be fetched: tag, size, address, key, id
  kOpSendTaken = 105,    // the receiver has fetched (or refused) the payload of offer `id`
  kOpErrorNotice = 102, // "this rank entered its error state because ...": the receivers enter theirs at once
                        // (the reference's ranks learn of a peer's error state only when that process exits)
};

struct TraceEvent {
  std::string name;
  int tid;
  double ts_us;
  double dur_us;
};

class HostGroup {
 public:
  static std::unique_ptr<HostGroup> create(KVStore& store, const std::string& key, int rank, int world);
  virtual ~HostGroup() = default;

  virtual int rank() const = 0;
  virtual int world() const = 0;
  virtual const std::string& name() const = 0;

  // ---- blocking CPU-tensor collectives (the caller's thread sleeps on a futex-like wait while the
  //      engine thread moves the data; reference: core/processgroup.cc:1088-1108) ----
  virtual void all_gather(const void* in, void* out, size_t bytes) = 0;
  virtual void reduce_scatter(const void* in, void* out, size_t count, int dtype, int op, double premul) = 0;
  virtual void all_reduce(const void* in, void* out, size_t count, int dtype, int op, double premul) = 0;
  virtual void broadcast(void* data, size_t bytes, int root) = 0;
  virtual void gather(const void* in, void* out, size_t bytes, int root) = 0;
  virtual void scatter(const void* in, void* out, size_t bytes, int root) = 0;
  virtual void all_to_all(const void* in, void* out, const uint64_t* send_off, const uint64_t* send_bytes,
                          const uint64_t* recv_off, const uint64_t* recv_bytes) = 0;
  virtual void barrier() = 0;
  virtual void send(const void* data, size_t bytes, int dst, uint32_t tag) = 0;
  virtual void recv(void* data, size_t bytes, int src, uint32_t tag) = 0;
  // The send in two steps. Small payloads travel inside their message and the returned request is complete at
  // once; a large one is offered to the receiver, which fetches it straight out of the caller's memory (one copy,
  // made by the receiving process where the two share a machine) once a matching receive exists, so the memory
  // (held through `keep`) must stay unchanged until send_wait() returns.
  virtual std::shared_ptr<void> send_post(const void* data, size_t bytes, int dst, uint32_t tag, std::shared_ptr<void> keep) = 0;
  virtual void send_wait(const std::shared_ptr<void>& posted) = 0;
  virtual bool send_done(const std::shared_ptr<void>& posted) = 0;
  // The receive in two steps: recv_post() files the request and returns at once (requests from one source with one
  // tag are served in the order they were posted; `keep` is held until the data has landed, so the destination
  // cannot go away under it), recv_wait() blocks until it is served and raises what went wrong.
  virtual std::shared_ptr<void> recv_post(void* data, size_t bytes, int src, uint32_t tag, std::shared_ptr<void> keep) = 0;
  virtual void recv_wait(const std::shared_ptr<void>& posted) = 0;
  virtual bool recv_done(const std::shared_ptr<void>& posted) = 0;
  // `src` = -1 in recv_post takes the first matching message of any rank; after recv_wait this says whose it was.
  virtual int recv_source(const std::shared_ptr<void>& posted) = 0;

  // ---- two-sided engine messages for subsystems layered on top (Queue, compile_op) ----
  using Handler = std::function<void(int src, Reader& body)>;  // runs on the engine thread
  virtual void set_handler(uint32_t op, Handler h) = 0;
  // several at once: messages of these types that came early are then replayed in the order they arrived in
  virtual void set_handlers(std::vector<std::pair<uint32_t, Handler>> handlers) = 0;
  virtual void send_message(int dst, uint32_t op, Bytes body) = 0;
  // Post a closure to the engine thread.
  virtual void run_on_engine(std::function<void()> fn) = 0;
  // A place for subsystems layered on the group to keep per-group state that must die with it (looked up by
  // name; the reference is valid for the life of the group, the caller synchronises its own use of the object).
  virtual std::shared_ptr<void>& extension(const std::string& key) = 0;
  virtual bool on_engine_thread() const = 0;
  // One-sided read of a peer's registered memory (engine thread only). Register with MrTable.
  virtual void post_read(int src, void* local, size_t bytes, uint32_t rkey, uint64_t raddr,
                         std::function<void(bool ok)> done) = 0;
  // The same for `rows` runs of `row_bytes` bytes, `src_pitch` apart at the peer, `dst_pitch` apart locally:
  // one request, one reply.
  virtual void post_read_strided(int src, void* local, uint64_t rows, size_t row_bytes, size_t dst_pitch, uint32_t rkey,
                                 uint64_t raddr, size_t src_pitch, std::function<void(bool ok)> done) = 0;

  // ---- health ----
  // {payload+header bytes sent over TCP, received over TCP, payload bytes copied directly between address
  // spaces of this machine, number of peers this rank reads directly}
  virtual std::vector<uint64_t> transport_counters() = 0;
  // Host-side fault injection for tests, applied to the two-sided engine messages this rank sends from now on:
  // every `drop_every`-th is dropped, every `duplicate_every`-th is sent twice, and each one is held back for
  // `delay_ms` first (0 switches a kind off). One-sided payload transfers are not touched.
  virtual void inject_faults(int drop_every, int duplicate_every, int delay_ms) = 0;
  virtual bool in_error() const = 0;
  virtual std::string error_text() const = 0;
  virtual void shutdown() = 0;  // coordinated: tells every peer, waits briefly for theirs

  // ---- profiling (reference: core/cputhread.cc:1008-1078) ----
  virtual void set_profiling(bool on) = 0;  // switching off writes moodist-trace-cpu-<group>-<rank>.json
  virtual bool profiling() const = 0;
  virtual std::string last_trace_path() const = 0;
};

}  // namespace moodist
