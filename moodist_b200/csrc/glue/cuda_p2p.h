// CUDA tensors handed from one rank to another without blocking the sender's host thread: Queue items and
// send / recv.
//
// The sender makes the bytes readable by its peers — in place when the tensor already lives in the symmetric
// heap, else through a stream-ordered copy into a heap buffer — queues a one-warp kernel that raises a flag
// word once the stream gets there, and posts a small descriptor (source rank, heap offset, size, flag) through
// the host path at once. Whoever receives the descriptor makes ITS stream wait for the flag (a bounded spin on
// the sender's memory through the peer mapping), copies the bytes over NVLink with a DMA copy, and lets a host
// callback on that stream tell the sender that the buffer is free again.
//
// The reference does the same hand-over with registered memory, a cuLaunchHostFunc trigger on the sender's
// stream and cuStreamWaitValue32 on the receiver's (core/queue.cc:629-696, 34-54); here the order of items
// follows the order of the put calls because the descriptor leaves immediately, and the device-side wait is
// bounded like every other wait of this library.
#pragma once

#include <ATen/ATen.h>
#include <cuda_runtime_api.h>

#include <map>
#include <mutex>

#include "core/host_group.h"

namespace moodist {

class CudaGroup;
class SymmHeap;

struct CudaItemDescriptor {
  uint64_t magic = 0;
  int32_t src_rank = -1;
  uint32_t buf_id = 0;
  uint64_t heap_off = 0;
  uint64_t bytes = 0;
  uint64_t flag_off = 0;
  uint32_t flag_val = 0;
  uint32_t reserved = 0;
};
constexpr uint64_t kCudaItemMagic = 0x6d6f6f6463756461ull;  // "moodcuda"

class CudaP2P {
 public:
  CudaP2P(CudaGroup& group, HostGroup& host, int device);
  ~CudaP2P();

  // Sender: publish `t` (contiguous) for `readers` receivers; `stream` is where `t` was produced.
  CudaItemDescriptor publish(const at::Tensor& t, int readers, cudaStream_t stream);
  // Receiver: stream-ordered copy of the published bytes into `dst` (d.bytes bytes), then the acknowledgement.
  void fetch(const CudaItemDescriptor& d, void* dst, cudaStream_t stream);
  // A descriptor that will never be fetched (a cancelled transaction): release what it holds.
  void drop(const CudaItemDescriptor& d);

  size_t held() const;

 private:
  struct Held {
    void* staged = nullptr;  // heap buffer to free, or
    at::Tensor keep;         // the heap-resident tensor itself
    int remaining = 0;
  };
  void release(uint32_t buf_id);

  CudaGroup& group_;
  HostGroup& host_;
  SymmHeap& heap_;
  int device_;
  uint32_t* flags_ = nullptr;  // 1024 words in the symmetric heap
  mutable std::mutex mu_;
  std::map<uint32_t, Held> held_;
  uint32_t next_buf_ = 0;
  uint32_t next_flag_val_ = 0;
};

}  // namespace moodist
