// Node topology as the collectives need it: which GPUs exist, which pairs can address each other's memory
// and over what (NVLink through NVSwitch, direct NVLink, PCIe), how many NVLink links are up, and which NUMA
// node each GPU hangs off. The probe is an interface so that tests (and hosts without a GPU) can feed a
// recorded machine instead of NVML.
//
// The reference discovers the same facts in core/group.cc (NVML P2P matrix, PCI bus ids exchanged between
// ranks, NUMA node per device used to pin its threads and pick NICs, core/group.cc:120-420); here they are
// gathered once per process and exchanged over the bootstrap ring when a group is created.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace moodist {

enum class LinkKind : int { None = 0, Pcie = 1, NvLink = 2, Self = 3 };

struct GpuInfo {
  int index = -1;            // NVML / CUDA index on this host
  std::string pci_bus_id;    // "0000:1b:00.0" (lower case)
  int numa_node = -1;        // -1 unknown
  int nvlinks_up = 0;        // active NVLink links
  int nvlinks_to_switch = 0; // of those, links whose remote end is not a GPU (an NVSwitch)
};

// What the machine can be asked. Every call returns false / -1 when the fact is unavailable.
class TopologyProbe {
 public:
  virtual ~TopologyProbe() = default;
  virtual int device_count() = 0;
  virtual bool pci_bus_id(int dev, std::string* out) = 0;
  virtual int numa_node(int dev) = 0;
  virtual int max_links() { return 18; }
  virtual bool link_up(int dev, int link) = 0;
  // PCI bus id of whatever sits at the other end of the link ("" when unknown)
  virtual bool link_remote(int dev, int link, std::string* pci) = 0;
  // 1 when dev_a can read / write dev_b's memory
  virtual int p2p_ok(int dev_a, int dev_b) = 0;
};

std::unique_ptr<TopologyProbe> make_nvml_probe();  // null when NVML is not loadable

struct NodeTopology {
  std::string node_id;  // boot id of this host: equal on two ranks <=> same machine
  std::vector<GpuInfo> gpus;
  std::vector<std::vector<LinkKind>> link;  // [a][b]
  bool nvswitch = false;                    // every GPU reaches every other through switch links
  bool all_p2p = false;

  std::string describe() const;
  std::vector<uint8_t> encode() const;
  static NodeTopology decode(const std::vector<uint8_t>& bytes);
};

NodeTopology discover_topology(TopologyProbe& probe);
// Cached discovery through NVML (an empty topology with only node_id when there is no NVML).
const NodeTopology& local_topology();

// A group's view: which ranks share this rank's machine, and whether the device kernels can be used among them.
struct GroupTopology {
  std::vector<int> local_ranks;     // ranks on this machine, ascending (includes this rank)
  std::vector<std::string> node_of; // node id per rank
  int num_nodes = 1;
  bool single_node = true;
  bool kernels_usable = true;       // single node and every pair of used GPUs can address each other
  std::string why_not;              // reason when kernels_usable is false
};
// node_ids / devices: per rank, as exchanged at group creation (device -1: CPU-only rank).
GroupTopology make_group_topology(int rank, const std::vector<std::string>& node_ids, const std::vector<int>& devices,
                                  const NodeTopology& local);

std::string read_boot_id();
int numa_node_of_pci(const std::string& pci_bus_id);  // from sysfs, -1 when unknown

}  // namespace moodist
