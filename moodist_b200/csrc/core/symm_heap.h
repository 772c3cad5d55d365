// Symmetric heap: this process's registered device memory, visible to every peer process on the node.
//
// One heap per (process, device). It owns a large reserved virtual range into which physical chunks
// (cuMemCreate, POSIX-fd shareable) are mapped back to back. Every chunk is exported once and imported
// by every known peer into that peer's *mirror* range for this process at the same offset, so
//     peer_address = mirror_base(peer) + (ptr - heap_base)
// holds for any pointer in the heap. Chunk fds travel over an abstract Unix socket served by a helper
// thread in each process (SCM_RIGHTS), which maps the chunk and acknowledges; growth is therefore
// possible at any time without a collective call.
//
// Group resources (flag page + staging area) are dedicated chunks so they can also be bound to an NVLS
// multicast object (cuMulticastCreate / AddDevice / BindMem), giving one address that stores to every
// GPU's copy and loads the switch-reduced sum.
//
// This replaces the reference's IpcMapper (core/ipc_mapper.cc:16-557: per-tensor cuIpc handles opened
// lazily by a peer-side thread through shared-memory request slots) and its CUDA allocator
// (core/allocator.cc:547-672: cuMemAlloc'd regions shared whole via owns/mappedRegion).
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "kvstore.h"

namespace moodist {

struct GroupMemory {
  // all addresses valid on the local device
  std::vector<void*> heap_base;     // [world] base of each rank's heap (own heap for `rank`)
  std::vector<void*> stage;         // [world] staging area of each rank
  std::vector<uint32_t*> flags;     // [world] flag page of each rank
  size_t staging_bytes = 0;
  void* mc_stage = nullptr;         // multicast alias of the staging areas (null without NVLS)
  uint32_t* mc_flags = nullptr;     // multicast alias of the flag pages
  uint32_t* status = nullptr;       // local status word (lives in the local flag chunk, after the flags)
};

class SymmHeap {
 public:
  // The heap of the calling thread's current device (created on first use).
  static SymmHeap& instance(int device);
  // True once instance(device) has been created (the allocator hooks use this).
  static bool exists(int device);

  virtual ~SymmHeap() = default;
  virtual int device() const = 0;
  virtual void* base() const = 0;
  virtual size_t reserved_bytes() const = 0;
  virtual size_t mapped_bytes() const = 0;
  virtual size_t allocated_bytes() const = 0;

  // Sub-allocation for the CUDA allocator hooks. Thread safe. Returns nullptr when out of memory.
  virtual void* alloc(size_t bytes) = 0;
  virtual void free(void* p) = 0;
  // Byte offset inside the heap, or -1 when [p, p+bytes) is not heap memory.
  virtual int64_t offset_of(const void* p, size_t bytes) const = 0;

  // Collective over the group (rendezvous through `store`): makes every member a known peer, creates
  // this rank's flag page + staging chunk, learns everyone else's, optionally builds the NVLS alias.
  virtual GroupMemory attach_group(KVStore& store, const std::string& group_key, int rank, int world,
                                   size_t staging_bytes, bool want_nvls) = 0;
  // Releases the group's chunk (peers keep their mapping until they exit).
  virtual void detach_group(const std::string& group_key) = 0;

  // Diagnostics
  virtual std::string describe() const = 0;
};

// One request of the heap's peer-to-peer channel: connect to the abstract Unix socket `sock` (retrying for at
// most `connect_seconds`: a refused connection means nobody listens there), send `bytes` bytes of `msg` with the
// file descriptor `fd` attached, and wait for the peer's 4-byte status. True only when the peer answered 0.
bool heap_request(const std::string& sock, const void* msg, size_t bytes, int fd, double connect_seconds);

}  // namespace moodist
