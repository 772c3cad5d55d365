#include "cpu_allocator.h"

#include <sys/mman.h>

#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "log.h"

namespace moodist {
namespace {

constexpr size_t kMinClass = 6;                 // 64 B
constexpr size_t kMaxClass = 28;                // 256 MiB; larger requests get their own mapping
constexpr size_t kRegionBytes = 1ull << 30;     // arenas of 1 GiB of address space (committed on touch)
constexpr size_t kSlabBytes = 16ull << 20;      // a size class grows by at least 16 MiB at a time

struct Header {  // sits 64 bytes before every block
  uint64_t magic;
  uint32_t cls;
  uint32_t direct;   // 1: own mapping of `mapped` bytes
  uint64_t mapped;
  uint64_t pad[5];
};
static_assert(sizeof(Header) == 64, "header keeps blocks 64-byte aligned");
constexpr uint64_t kMagic = 0x6d6f6f5f63707521ull;

struct Region {
  uint8_t* base;
  size_t size, used;
};

struct State {
  std::mutex mu;
  std::vector<Region> regions;
  std::vector<void*> free_lists[kMaxClass + 1];
  std::map<uintptr_t, size_t> spans;  // every mapping we made: base -> size
  uint64_t live[kMaxClass + 1] = {}, total[kMaxClass + 1] = {};
  uint64_t direct_live = 0, direct_bytes = 0;
};
State& st() {
  static State* s = new State();
  return *s;
}

void* map_bytes(size_t n) {
  void* p = mmap(nullptr, n, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  return p == MAP_FAILED ? nullptr : p;
}

// carve `bytes` out of the current arena (new arena when it is full)
uint8_t* carve(State& s, size_t bytes) {
  if (s.regions.empty() || s.regions.back().used + bytes > s.regions.back().size) {
    size_t n = bytes > kRegionBytes ? bytes : kRegionBytes;
    uint8_t* base = (uint8_t*)map_bytes(n);
    if (!base) return nullptr;
    s.regions.push_back(Region{base, n, 0});
    s.spans[(uintptr_t)base] = n;
  }
  Region& r = s.regions.back();
  uint8_t* p = r.base + r.used;
  r.used += bytes;
  return p;
}

}  // namespace

void* cpu_alloc(size_t bytes) {
  State& s = st();
  size_t need = bytes + sizeof(Header);
  size_t cls = kMinClass;
  while (cls <= kMaxClass && ((size_t)1 << cls) < need) ++cls;
  std::lock_guard<std::mutex> lk(s.mu);
  if (cls > kMaxClass) {
    size_t n = (need + 4095) & ~(size_t)4095;
    uint8_t* base = (uint8_t*)map_bytes(n);
    if (!base) return nullptr;
    s.spans[(uintptr_t)base] = n;
    Header* h = (Header*)base;
    *h = Header{kMagic, 0, 1, n, {}};
    ++s.direct_live;
    s.direct_bytes += n;
    return base + sizeof(Header);
  }
  auto& fl = s.free_lists[cls];
  if (fl.empty()) {
    size_t block = (size_t)1 << cls;
    size_t slab = block > kSlabBytes ? block : kSlabBytes;
    uint8_t* p = carve(s, slab);
    if (!p) return nullptr;
    for (size_t off = 0; off + block <= slab; off += block) fl.push_back(p + off);
    s.total[cls] += slab / block;
  }
  uint8_t* blk = (uint8_t*)fl.back();
  fl.pop_back();
  Header* h = (Header*)blk;
  *h = Header{kMagic, (uint32_t)cls, 0, 0, {}};
  ++s.live[cls];
  return blk + sizeof(Header);
}

void cpu_free(void* p) {
  if (!p) return;
  State& s = st();
  Header* h = (Header*)((uint8_t*)p - sizeof(Header));
  if (h->magic != kMagic) {
    log_error("moodist CPU allocator: free of a pointer it does not own (%p)", p);
    return;
  }
  std::lock_guard<std::mutex> lk(s.mu);
  h->magic = 0;  // catches double frees
  if (h->direct) {
    size_t n = h->mapped;
    s.spans.erase((uintptr_t)h);
    --s.direct_live;
    s.direct_bytes -= n;
    munmap(h, n);
    return;
  }
  --s.live[h->cls];
  s.free_lists[h->cls].push_back(h);
}

bool cpu_allocator_region(const void* p, void** base, size_t* size) {
  State& s = st();
  std::lock_guard<std::mutex> lk(s.mu);
  auto it = s.spans.upper_bound((uintptr_t)p);
  if (it == s.spans.begin()) return false;
  --it;
  if ((uintptr_t)p >= it->first + it->second) return false;
  if (base) *base = (void*)it->first;
  if (size) *size = it->second;
  return true;
}

bool cpu_allocator_owns(const void* p) { return cpu_allocator_region(p, nullptr, nullptr); }

std::string cpu_allocator_debug() {
  State& s = st();
  std::lock_guard<std::mutex> lk(s.mu);
  std::string out = strf("moodist CPU allocator: %zu arenas\n", s.regions.size());
  for (size_t c = kMinClass; c <= kMaxClass; ++c)
    if (s.total[c])
      out += strf("  class %2zu (%10zu B): %llu live / %llu blocks\n", c, (size_t)1 << c, (unsigned long long)s.live[c],
                  (unsigned long long)s.total[c]);
  out += strf("  direct mappings: %llu live, %llu bytes\n", (unsigned long long)s.direct_live, (unsigned long long)s.direct_bytes);
  return out;
}

}  // namespace moodist
