// CPU allocator for tensors that travel through the engine: power-of-two size classes carved out of large
// mmap'd regions, so that the transport can register a whole region once (one MrTable entry, one
// cuMemHostRegister) instead of every tensor. Reference: core/cpu_allocator.cc:165-385, 418-497, 583-617.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

namespace moodist {

void* cpu_alloc(size_t bytes);
void cpu_free(void* p);
// True when `p` points into memory handed out by cpu_alloc.
bool cpu_allocator_owns(const void* p);
// The mapped region around `p` (for one-off registration); false if not ours.
bool cpu_allocator_region(const void* p, void** base, size_t* size);
// Human-readable usage per size class (moodist.cpu_allocator_debug()).
std::string cpu_allocator_debug();

}  // namespace moodist
