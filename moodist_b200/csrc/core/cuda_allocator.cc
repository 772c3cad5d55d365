// Registered-memory CUDA allocator: device memory for torch tensors comes out of the symmetric heap, so
// every tensor is already mapped at every peer and collectives read it in place (no staging copy, NVLS
// eligible). Exposed to torch through its pluggable-allocator hooks (mb_cuda_alloc / mb_cuda_free).
//
// Reuse policy, after the reference's allocator (core/allocator.cc:674-738, 847-923): a freed block is
// immediately reusable by the stream that freed it (stream order protects it); for any other stream it
// becomes available once an event recorded at the free point has completed, so no allocation ever
// synchronises the device. Blocks are cached per (stream, size); the cache is trimmed back into the heap
// when the heap cannot satisfy a request.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <deque>
#include <map>
#include <mutex>
#include <unordered_map>

#include "log.h"
#include "symm_heap.h"

namespace moodist {
namespace {

struct Freed {
  void* ptr;
  size_t size;
  cudaStream_t stream;
  cudaEvent_t event;
};

struct DeviceCache {
  std::mutex mu;
  std::map<std::pair<cudaStream_t, size_t>, std::deque<void*>> same_stream;  // reusable in stream order
  std::deque<Freed> pending;                                                 // waiting for their event
  std::deque<cudaEvent_t> spare_events;
  std::unordered_map<void*, size_t> live;
  uint64_t hits = 0, misses = 0, bytes_live = 0, bytes_cached = 0;
};

DeviceCache& cache(int device) {
  static DeviceCache caches[64];
  return caches[device & 63];
}

size_t round_size(size_t n) {
  if (n < 512) return 512;
  if (n < (1u << 20)) return (n + 511) & ~(size_t)511;
  return (n + (2u << 20) - 1) & ~(size_t)((2u << 20) - 1);  // large blocks in 2 MiB steps: better reuse
}

// return finished blocks to the heap; with `all`, also the same-stream cache (after a device sync)
void trim(DeviceCache& c, SymmHeap& heap, bool all) {
  while (!c.pending.empty()) {
    Freed& f = c.pending.front();
    if (!all && cudaEventQuery(f.event) != cudaSuccess) break;
    heap.free(f.ptr);
    c.bytes_cached -= f.size;
    c.spare_events.push_back(f.event);
    c.pending.pop_front();
  }
  cudaGetLastError();
  if (all) {
    for (auto& [key, list] : c.same_stream) {
      for (void* p : list) {
        heap.free(p);
        c.bytes_cached -= key.second;
      }
    }
    c.same_stream.clear();
  }
}

}  // namespace
}  // namespace moodist

using namespace moodist;

extern "C" void* mb_cuda_alloc(ssize_t size, int device, cudaStream_t stream) {
  if (size <= 0) return nullptr;
  try {
    SymmHeap& heap = SymmHeap::instance(device);
    DeviceCache& c = cache(device);
    size_t n = round_size((size_t)size);
    std::lock_guard<std::mutex> lk(c.mu);
    auto it = c.same_stream.find({stream, n});
    if (it != c.same_stream.end() && !it->second.empty()) {
      void* p = it->second.back();
      it->second.pop_back();
      c.bytes_cached -= n;
      c.live[p] = n;
      c.bytes_live += n;
      ++c.hits;
      return p;
    }
    ++c.misses;
    trim(c, heap, false);
    void* p = heap.alloc(n);
    if (!p) {
      // out of memory: give everything cached back and try once more
      cudaDeviceSynchronize();
      trim(c, heap, true);
      p = heap.alloc(n);
    }
    if (!p) {
      log_error("moodist CUDA allocator: out of memory allocating %zu bytes (%s; live %llu MiB, cached %llu MiB)", n,
                heap.describe().c_str(), (unsigned long long)(c.bytes_live >> 20), (unsigned long long)(c.bytes_cached >> 20));
      return nullptr;
    }
    c.live[p] = n;
    c.bytes_live += n;
    return p;
  } catch (const std::exception& e) {
    log_error("moodist CUDA allocator: %s", e.what());
    return nullptr;
  }
}

extern "C" void mb_cuda_free(void* ptr, ssize_t /*size*/, int device, cudaStream_t stream) {
  if (!ptr) return;
  DeviceCache& c = cache(device);
  std::lock_guard<std::mutex> lk(c.mu);
  auto it = c.live.find(ptr);
  if (it == c.live.end()) {
    log_error("moodist CUDA allocator: free of a pointer it does not own: %p", ptr);
    return;
  }
  size_t n = it->second;
  c.live.erase(it);
  c.bytes_live -= n;
  c.bytes_cached += n;
  auto& list = c.same_stream[{stream, n}];
  if (list.size() < 8) {
    list.push_back(ptr);
    return;
  }
  // enough of this size cached for the stream: let the block go back to the heap once the stream passes here
  Freed f{ptr, n, stream, nullptr};
  if (!c.spare_events.empty()) {
    f.event = c.spare_events.back();
    c.spare_events.pop_back();
  } else if (cudaEventCreateWithFlags(&f.event, cudaEventDisableTiming) != cudaSuccess) {
    cudaGetLastError();
    list.push_back(ptr);
    return;
  }
  cudaEventRecord(f.event, stream);
  c.pending.push_back(f);
}

// {live bytes, cached bytes, hits, misses, heap mapped bytes}
extern "C" void mb_cuda_allocator_stats(int device, uint64_t* out5) {
  DeviceCache& c = cache(device);
  std::lock_guard<std::mutex> lk(c.mu);
  out5[0] = c.bytes_live;
  out5[1] = c.bytes_cached;
  out5[2] = c.hits;
  out5[3] = c.misses;
  out5[4] = SymmHeap::exists(device) ? SymmHeap::instance(device).mapped_bytes() : 0;
}
