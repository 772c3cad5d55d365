// Registered-memory CUDA allocator: device memory for torch tensors comes out of the symmetric heap, so
// every tensor is already mapped at every peer and collectives read it in place (no staging copy, NVLS
// eligible). Exposed to torch through its pluggable-allocator hooks (mb_cuda_alloc / mb_cuda_free).
//
// Reuse policy, after the reference's allocator (core/allocator.cc:674-738, 847-923): a freed block is
// immediately reusable by the stream that freed it (stream order protects it); for any other stream it
// becomes available once an event recorded at the free point has completed, so no allocation ever
// synchronises the device. Blocks are cached per (stream, size); the cache is trimmed back into the heap
// when the heap cannot satisfy a request.
// A block that was also used on other streams (torch calls record_stream for it, reference:
// core/allocator.cc:1219-1232, wrapper/allocator_wrapper.cc:92-100) is never handed back in stream order:
// when it is freed, one event is recorded on every stream that used it and the block returns to the heap
// only after all of them have completed.
// MOODIST_MEM_LOG_LEVEL (same values as MOODIST_LOG_LEVEL; reference: core/allocator.cc:16-70) turns on a line
// per heap allocation, trim and out-of-memory event (VERBOSE) or per alloc / free call (DEBUG).
#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstdint>
#include <deque>
#include <vector>
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
  std::vector<cudaEvent_t> events;  // one per stream that used the block; all must complete
};

struct Live {
  size_t size = 0;
  std::vector<cudaStream_t> streams;  // streams other than the allocating one that used the block
};

struct DeviceCache {
  std::mutex mu;
  std::map<std::pair<cudaStream_t, size_t>, std::deque<void*>> same_stream;  // reusable in stream order
  std::deque<Freed> pending;                                                 // waiting for their events
  std::deque<cudaEvent_t> spare_events;
  std::unordered_map<void*, Live> live;
  uint64_t hits = 0, misses = 0, bytes_live = 0, bytes_cached = 0, cross_stream_frees = 0;
};

int mem_log_level() {
  static int lvl = parse_log_level(getenv("MOODIST_MEM_LOG_LEVEL"), LOG_NONE);
  return lvl;
}
#define MEM_LOG(level, ...)                                   \
  do {                                                        \
    if (mem_log_level() >= (level)) {                         \
      std::string line_ = strf(__VA_ARGS__);                  \
      fprintf(stdout, "moodist mem: %s\n", line_.c_str());    \
      fflush(stdout);                                         \
    }                                                         \
  } while (0)

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
  size_t returned = 0;
  for (auto it = c.pending.begin(); it != c.pending.end();) {
    bool done = true;
    if (!all)
      for (cudaEvent_t e : it->events) done = done && cudaEventQuery(e) == cudaSuccess;
    if (!done) {
      ++it;
      continue;
    }
    heap.free(it->ptr);
    c.bytes_cached -= it->size;
    returned += it->size;
    for (cudaEvent_t e : it->events) c.spare_events.push_back(e);
    it = c.pending.erase(it);
  }
  cudaGetLastError();
  if (returned) MEM_LOG(LOG_VERBOSE, "trim returned %zu bytes to the heap (%zu blocks still wait for events)", returned, c.pending.size());
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
      c.live[p] = Live{n, {}};
      c.bytes_live += n;
      ++c.hits;
      MEM_LOG(LOG_DEBUG, "alloc %zu bytes on stream %p: cached block %p", n, (void*)stream, p);
      return p;
    }
    ++c.misses;
    trim(c, heap, false);
    void* p = heap.alloc(n);
    if (!p) {
      // out of memory: give everything cached back and try once more
      MEM_LOG(LOG_VERBOSE, "heap full at %zu bytes: synchronising and returning every cached block", n);
      cudaDeviceSynchronize();
      trim(c, heap, true);
      p = heap.alloc(n);
    }
    if (!p) {
      log_error("moodist CUDA allocator: out of memory allocating %zu bytes (%s; live %llu MiB, cached %llu MiB)", n,
                heap.describe().c_str(), (unsigned long long)(c.bytes_live >> 20), (unsigned long long)(c.bytes_cached >> 20));
      return nullptr;
    }
    c.live[p] = Live{n, {}};
    c.bytes_live += n;
    MEM_LOG(LOG_VERBOSE, "alloc %zu bytes on stream %p: new block %p (live %llu MiB, cached %llu MiB, %s)", n, (void*)stream, p,
            (unsigned long long)(c.bytes_live >> 20), (unsigned long long)(c.bytes_cached >> 20), heap.describe().c_str());
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
  size_t n = it->second.size;
  std::vector<cudaStream_t> streams = std::move(it->second.streams);
  c.live.erase(it);
  c.bytes_live -= n;
  c.bytes_cached += n;
  MEM_LOG(LOG_DEBUG, "free %p (%zu bytes) on stream %p, used on %zu other stream(s)", ptr, n, (void*)stream, streams.size());
  auto& list = c.same_stream[{stream, n}];
  if (streams.empty() && list.size() < 8) {
    list.push_back(ptr);
    return;
  }
  // Either enough of this size is cached for the stream, or other streams used the block: it goes back to the
  // heap once every stream that touched it has passed this point.
  if (!streams.empty()) ++c.cross_stream_frees;
  streams.push_back(stream);
  Freed f{ptr, n, {}};
  for (cudaStream_t s : streams) {
    cudaEvent_t e = nullptr;
    if (!c.spare_events.empty()) {
      e = c.spare_events.back();
      c.spare_events.pop_back();
    } else if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      // no event to be had: make the block safe the slow way
      cudaStreamSynchronize(s);
      continue;
    }
    cudaEventRecord(e, s);
    f.events.push_back(e);
  }
  c.pending.push_back(std::move(f));
}

// torch's Tensor.record_stream: the block is in use on `stream` too.
extern "C" void mb_cuda_record_stream(void* ptr, cudaStream_t stream) {
  if (!ptr) return;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return;
  // the block may belong to another device than the current one: look in every cache that knows it
  for (int d = 0; d < 64; ++d) {
    DeviceCache& c = cache((device + d) & 63);
    std::lock_guard<std::mutex> lk(c.mu);
    auto it = c.live.find(ptr);
    if (it == c.live.end()) continue;
    auto& v = it->second.streams;
    if (std::find(v.begin(), v.end(), stream) == v.end()) v.push_back(stream);
    return;
  }
}

// Base address and size of the allocation that contains `ptr` (every block is its own allocation here);
// nullptr when the allocator does not own it.
extern "C" void* mb_cuda_base_allocation(void* ptr, size_t* size) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
  for (int d = 0; d < 64; ++d) {
    DeviceCache& c = cache((device + d) & 63);
    std::lock_guard<std::mutex> lk(c.mu);
    for (auto& [base, info] : c.live) {
      if ((uintptr_t)ptr >= (uintptr_t)base && (uintptr_t)ptr < (uintptr_t)base + info.size) {
        if (size) *size = info.size;
        return base;
      }
    }
  }
  return nullptr;
}

// {live bytes, cached bytes, hits, misses, heap mapped bytes}; mb_cuda_allocator_stats6 adds the number of
// frees that had to wait for other streams
extern "C" uint64_t mb_cuda_allocator_cross_stream_frees(int device) {
  DeviceCache& c = cache(device);
  std::lock_guard<std::mutex> lk(c.mu);
  return c.cross_stream_frees;
}
extern "C" void mb_cuda_allocator_stats(int device, uint64_t* out5) {
  DeviceCache& c = cache(device);
  std::lock_guard<std::mutex> lk(c.mu);
  out5[0] = c.bytes_live;
  out5[1] = c.bytes_cached;
  out5[2] = c.hits;
  out5[3] = c.misses;
  out5[4] = SymmHeap::exists(device) ? SymmHeap::instance(device).mapped_bytes() : 0;
}
