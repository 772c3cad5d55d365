#include "numa.h"

#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cstdint>
#include <cstdlib>
#include <fstream>
#include <sstream>

#include "log.h"

namespace moodist {

std::vector<int> parse_cpu_list(const std::string& text) {
  std::vector<int> out;
  std::stringstream ss(text);
  std::string part;
  while (std::getline(ss, part, ',')) {
    while (!part.empty() && (part.back() == '\n' || part.back() == ' ')) part.pop_back();
    if (part.empty()) continue;
    size_t dash = part.find('-');
    try {
      if (dash == std::string::npos) {
        out.push_back(std::stoi(part));
      } else {
        int lo = std::stoi(part.substr(0, dash)), hi = std::stoi(part.substr(dash + 1));
        for (int c = lo; c <= hi && c - lo < 4096; ++c) out.push_back(c);
      }
    } catch (...) {
      return {};
    }
  }
  return out;
}

int numa_node_count() {
  std::ifstream f("/sys/devices/system/node/online");
  std::string s;
  if (!f || !std::getline(f, s)) return 1;
  auto nodes = parse_cpu_list(s);
  return nodes.empty() ? 1 : (int)nodes.size();
}

std::vector<int> cpus_of_numa_node(int node) {
  if (node < 0) return {};
  std::ifstream f("/sys/devices/system/node/node" + std::to_string(node) + "/cpulist");
  std::string s;
  if (!f || !std::getline(f, s)) return {};
  return parse_cpu_list(s);
}

bool numa_binding_enabled() { return env_long("MOODIST_NUMA_BIND", 1) != 0; }

bool bind_thread_to_numa_node(int node) {
  if (!numa_binding_enabled()) return false;
  std::vector<int> cpus = cpus_of_numa_node(node);
  if (cpus.empty()) return false;
  cpu_set_t set;
  CPU_ZERO(&set);
  for (int c : cpus)
    if (c >= 0 && c < CPU_SETSIZE) CPU_SET(c, &set);
  // keep only CPUs this process may use at all (containers restrict the mask)
  cpu_set_t allowed;
  if (sched_getaffinity(0, sizeof(allowed), &allowed) == 0) {
    cpu_set_t both;
    CPU_AND(&both, &set, &allowed);
    if (CPU_COUNT(&both) == 0) return false;
    set = both;
  }
  return sched_setaffinity(0, sizeof(set), &set) == 0;
}

bool prefer_numa_node(void* p, size_t bytes, int node, bool move) {
  if (!numa_binding_enabled() || node < 0 || node >= 1024 || !p || !bytes) return false;
#ifdef SYS_mbind
  constexpr int kPreferred = 1;     // MPOL_PREFERRED
  constexpr unsigned kMove = 1u << 1;  // MPOL_MF_MOVE
  unsigned long mask[16] = {0};
  mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
  uintptr_t start = (uintptr_t)p & ~(uintptr_t)4095;
  size_t len = ((uintptr_t)p + bytes - start + 4095) & ~(size_t)4095;
  long rc = syscall(SYS_mbind, (void*)start, len, kPreferred, mask, (unsigned long)(8 * sizeof(mask)), move ? kMove : 0u);
  return rc == 0;
#else
  (void)move;
  return false;
#endif
}

}  // namespace moodist
