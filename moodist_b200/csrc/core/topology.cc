#include "topology.h"

#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <set>

#include "cuda_loader.h"
#include "log.h"
#include "wire.h"

namespace moodist {

namespace {

std::string lower(std::string s) {
  for (auto& ch : s) ch = (char)tolower((unsigned char)ch);
  return s;
}

// NVML's nvmlPciInfo_t as far as it is used here: busIdLegacy[16], domain, bus, device, pciDeviceId,
// pciSubSystemId, busId[32]
struct PciInfo {
  char bus_id_legacy[16];
  unsigned domain, bus, device, pci_device_id, pci_subsystem_id;
  char bus_id[32];
};

class NvmlProbe final : public TopologyProbe {
 public:
  explicit NvmlProbe(const NvmlApi& api) : n_(api) {}
  int device_count() override {
    unsigned c = 0;
    if (!n_.nvmlDeviceGetCount_v2 || n_.nvmlDeviceGetCount_v2(&c) != 0) return 0;
    return (int)c;
  }
  void* handle(int dev) {
    void* h = nullptr;
    if (!n_.nvmlDeviceGetHandleByIndex_v2 || n_.nvmlDeviceGetHandleByIndex_v2((unsigned)dev, &h) != 0) return nullptr;
    return h;
  }
  bool pci_bus_id(int dev, std::string* out) override {
    void* h = handle(dev);
    if (h && n_.nvmlDeviceGetPciInfo_v3) {
      PciInfo info;
      memset(&info, 0, sizeof(info));
      if (n_.nvmlDeviceGetPciInfo_v3(h, &info) == 0) {
        info.bus_id[31] = 0;
        *out = lower(info.bus_id);
        return true;
      }
    }
    // fall back to the driver's /proc listing, which sorts like NVML's indices (by PCI bus id)
    std::vector<std::string> ids = sysfs_nvidia_gpus();
    if (dev < 0 || dev >= (int)ids.size()) return false;
    *out = ids[dev];
    return true;
  }
  int numa_node(int dev) override {
    void* h = handle(dev);
    unsigned node = 0;
    if (h && n_.nvmlDeviceGetNumaNodeId && n_.nvmlDeviceGetNumaNodeId(h, &node) == 0) return (int)node;
    std::string pci;
    if (pci_bus_id(dev, &pci)) return numa_node_of_pci(pci);
    return -1;
  }
  bool link_up(int dev, int link) override {
    void* h = handle(dev);
    int active = 0;
    if (!h || !n_.nvmlDeviceGetNvLinkState) return false;
    return n_.nvmlDeviceGetNvLinkState(h, (unsigned)link, &active) == 0 && active == 1;
  }
  bool link_remote(int dev, int link, std::string* pci) override {
    void* h = handle(dev);
    PciInfo info;
    memset(&info, 0, sizeof(info));
    if (!h || !n_.nvmlDeviceGetNvLinkRemotePciInfo_v2) return false;
    if (n_.nvmlDeviceGetNvLinkRemotePciInfo_v2(h, (unsigned)link, &info) != 0) return false;
    info.bus_id[31] = 0;
    *pci = lower(info.bus_id);
    return true;
  }
  int p2p_ok(int a, int b) override {
    void *ha = handle(a), *hb = handle(b);
    int status = -1;
    // index 0 = read, 1 = write; status 0 = OK
    if (!ha || !hb || !n_.nvmlDeviceGetP2PStatus) return -1;
    if (n_.nvmlDeviceGetP2PStatus(ha, hb, 0, &status) != 0) return -1;
    if (status != 0) return 0;
    if (n_.nvmlDeviceGetP2PStatus(ha, hb, 1, &status) != 0) return -1;
    return status == 0 ? 1 : 0;
  }

  static std::vector<std::string> sysfs_nvidia_gpus() {
    // /proc/driver/nvidia/gpus/<bus id>/ exists per GPU the driver manages
    std::vector<std::string> out;
    if (auto* d = opendir_("/proc/driver/nvidia/gpus")) {
      while (auto* name = readdir_(d)) {
        std::string s = name;
        if (s.size() >= 7 && s[0] != '.') out.push_back(lower(s));
      }
      closedir_(d);
    }
    std::sort(out.begin(), out.end());
    return out;
  }

 private:
  // thin wrappers so <dirent.h> stays local to this file
  static void* opendir_(const char* path);
  static const char* readdir_(void* d);
  static void closedir_(void* d);
  const NvmlApi& n_;
};

}  // namespace
}  // namespace moodist

#include <dirent.h>
namespace moodist {
namespace {
void* NvmlProbe::opendir_(const char* path) { return opendir(path); }
const char* NvmlProbe::readdir_(void* d) {
  struct dirent* e = readdir((DIR*)d);
  return e ? e->d_name : nullptr;
}
void NvmlProbe::closedir_(void* d) { closedir((DIR*)d); }
}  // namespace

std::unique_ptr<TopologyProbe> make_nvml_probe() {
  const NvmlApi& api = nvml();
  if (!api.loaded) return nullptr;
  return std::make_unique<NvmlProbe>(api);
}

std::string read_boot_id() {
  std::ifstream f("/proc/sys/kernel/random/boot_id");
  std::string id;
  if (f && std::getline(f, id) && !id.empty()) return id;
  char host[256] = {0};
  gethostname(host, sizeof(host) - 1);
  return std::string("host:") + host;
}

int numa_node_of_pci(const std::string& pci_bus_id) {
  std::string id = lower(pci_bus_id);
  // NVML prints an 8-digit domain, sysfs a 4-digit one
  if (id.size() > 12 && id.compare(0, 4, "0000") == 0 && id[8] == ':') id = id.substr(4);
  std::ifstream f("/sys/bus/pci/devices/" + id + "/numa_node");
  int node = -1;
  if (f) f >> node;
  return node;
}

NodeTopology discover_topology(TopologyProbe& probe) {
  NodeTopology t;
  t.node_id = read_boot_id();
  int n = probe.device_count();
  if (n < 0) n = 0;
  t.gpus.resize(n);
  std::map<std::string, int> by_pci;
  for (int i = 0; i < n; ++i) {
    GpuInfo& g = t.gpus[i];
    g.index = i;
    probe.pci_bus_id(i, &g.pci_bus_id);
    g.pci_bus_id = lower(g.pci_bus_id);
    g.numa_node = probe.numa_node(i);
    if (!g.pci_bus_id.empty()) by_pci[g.pci_bus_id] = i;
  }
  // direct GPU<->GPU links and links that end in a switch
  std::vector<std::vector<int>> direct(n, std::vector<int>(n, 0));
  for (int i = 0; i < n; ++i) {
    for (int l = 0; l < probe.max_links(); ++l) {
      if (!probe.link_up(i, l)) continue;
      ++t.gpus[i].nvlinks_up;
      std::string remote;
      bool known = probe.link_remote(i, l, &remote);
      auto it = known ? by_pci.find(lower(remote)) : by_pci.end();
      if (it != by_pci.end()) {
        ++direct[i][it->second];
      } else {
        ++t.gpus[i].nvlinks_to_switch;
      }
    }
  }
  t.link.assign(n, std::vector<LinkKind>(n, LinkKind::None));
  t.all_p2p = n > 0;
  t.nvswitch = n > 1;
  for (int a = 0; a < n; ++a) {
    for (int b = 0; b < n; ++b) {
      if (a == b) {
        t.link[a][b] = LinkKind::Self;
        continue;
      }
      int ok = probe.p2p_ok(a, b);
      if (ok == 0) {  // an explicit "no"; when the machine does not answer (-1) the pair is not ruled out
        t.all_p2p = false;
        t.nvswitch = false;
        continue;
      }
      if (direct[a][b] > 0 || (t.gpus[a].nvlinks_to_switch > 0 && t.gpus[b].nvlinks_to_switch > 0)) {
        t.link[a][b] = LinkKind::NvLink;
      } else {
        t.link[a][b] = LinkKind::Pcie;
      }
      if (!(t.gpus[a].nvlinks_to_switch > 0 && t.gpus[b].nvlinks_to_switch > 0)) t.nvswitch = false;
    }
  }
  return t;
}

const NodeTopology& local_topology() {
  static NodeTopology topo;
  static std::once_flag once;
  std::call_once(once, [] {
    auto probe = make_nvml_probe();
    if (probe) {
      topo = discover_topology(*probe);
    } else {
      topo.node_id = read_boot_id();
    }
  });
  return topo;
}

std::string NodeTopology::describe() const {
  std::string s = strf("node %s: %d GPU(s), nvswitch=%d, all_p2p=%d\n", node_id.c_str(), (int)gpus.size(), (int)nvswitch,
                       (int)all_p2p);
  for (auto& g : gpus)
    s += strf("  gpu %d pci %s numa %d nvlinks %d (to switch %d)\n", g.index, g.pci_bus_id.c_str(), g.numa_node,
              g.nvlinks_up, g.nvlinks_to_switch);
  static const char* names[] = {"-", "PCIe", "NV", "self"};
  for (size_t a = 0; a < link.size(); ++a) {
    s += "  ";
    for (size_t b = 0; b < link[a].size(); ++b) s += strf("%5s", names[(int)link[a][b]]);
    s += "\n";
  }
  return s;
}

std::vector<uint8_t> NodeTopology::encode() const {
  std::vector<std::vector<int32_t>> links;
  for (auto& row : link) {
    std::vector<int32_t> r;
    for (auto k : row) r.push_back((int32_t)k);
    links.push_back(r);
  }
  std::vector<std::string> pcis;
  std::vector<int32_t> numa, up, sw;
  for (auto& g : gpus) {
    pcis.push_back(g.pci_bus_id);
    numa.push_back(g.numa_node);
    up.push_back(g.nvlinks_up);
    sw.push_back(g.nvlinks_to_switch);
  }
  return moodist::encode(node_id, pcis, numa, up, sw, links, nvswitch, all_p2p);
}

NodeTopology NodeTopology::decode(const std::vector<uint8_t>& bytes) {
  NodeTopology t;
  std::vector<std::vector<int32_t>> links;
  std::vector<std::string> pcis;
  std::vector<int32_t> numa, up, sw;
  decode_exact(bytes, t.node_id, pcis, numa, up, sw, links, t.nvswitch, t.all_p2p);
  if (numa.size() != pcis.size() || up.size() != pcis.size() || sw.size() != pcis.size() || links.size() != pcis.size())
    throw WireError("topology: inconsistent array lengths");
  t.gpus.resize(pcis.size());
  for (size_t i = 0; i < pcis.size(); ++i) {
    t.gpus[i].index = (int)i;
    t.gpus[i].pci_bus_id = pcis[i];
    t.gpus[i].numa_node = numa[i];
    t.gpus[i].nvlinks_up = up[i];
    t.gpus[i].nvlinks_to_switch = sw[i];
  }
  for (auto& r : links) {
    if (r.size() != pcis.size()) throw WireError("topology: link matrix is not square");
    std::vector<LinkKind> row;
    for (auto k : r) row.push_back((LinkKind)k);
    t.link.push_back(row);
  }
  return t;
}

GroupTopology make_group_topology(int rank, const std::vector<std::string>& node_ids, const std::vector<int>& devices,
                                  const NodeTopology& local) {
  GroupTopology g;
  g.node_of = node_ids;
  std::set<std::string> nodes(node_ids.begin(), node_ids.end());
  g.num_nodes = (int)nodes.size();
  g.single_node = g.num_nodes == 1;
  for (int r = 0; r < (int)node_ids.size(); ++r)
    if (node_ids[r] == node_ids[rank]) g.local_ranks.push_back(r);
  g.kernels_usable = true;
  if (!g.single_node) {
    g.kernels_usable = false;
    g.why_not = strf("ranks are spread over %d machines; the device kernels address peer memory inside one machine", g.num_nodes);
    return g;
  }
  std::set<int> used;
  for (int r : g.local_ranks) {
    int d = devices[r];
    if (d < 0) continue;
    if (!used.insert(d).second) {
      g.kernels_usable = false;
      g.why_not = strf("two ranks share GPU %d: kernels that wait on one another must not share a device", d);
      return g;
    }
  }
  for (int a : used)
    for (int b : used) {
      if (a == b || a >= (int)local.link.size() || b >= (int)local.link.size()) continue;
      if (local.link[a][b] == LinkKind::None) {
        g.kernels_usable = false;
        g.why_not = strf("GPU %d cannot address the memory of GPU %d", a, b);
        return g;
      }
    }
  return g;
}

}  // namespace moodist
