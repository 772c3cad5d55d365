// NUMA placement helpers: pin a thread to the CPUs of the memory node a GPU hangs off, and prefer that node
// for a range of host memory (staging buffers, allocator regions). Plain sysfs + syscalls, no libnuma.
// The reference does the same with libnuma-style calls for its engine threads and pinned buffers
// (core/group.cc NUMA node per device, core/cputhread.cc thread affinity).
#pragma once

#include <cstddef>
#include <string>
#include <vector>

namespace moodist {

int numa_node_count();                           // 1 on hosts without NUMA information
std::vector<int> cpus_of_numa_node(int node);    // empty when unknown
std::vector<int> parse_cpu_list(const std::string& text);  // "0-3,8,10-11" -> {0,1,2,3,8,10,11}
// Restrict the calling thread to the node's CPUs. false when the node is unknown or the call is refused.
bool bind_thread_to_numa_node(int node);
// Ask the kernel to place (and, with `move`, migrate) the pages of [p, p+bytes) on `node`. false if refused.
bool prefer_numa_node(void* p, size_t bytes, int node, bool move = false);
// MOODIST_NUMA_BIND=0 disables both bindings (default on).
bool numa_binding_enabled();

}  // namespace moodist
