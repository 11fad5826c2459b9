// Topology of the box as the plugin needs it: the GPUs, how each pair is connected (NVLink through
// NVSwitch, PCIe, nothing), the copy channels ("rails") that form each GPU's virtual NIC group, and
// an NCCL topology XML that places one virtual NIC next to each GPU so NCCL pairs GPU i with net
// device i (reference: src/nccl_ofi_topo.cpp — NIC/GPU grouping :884-1259, XML writer :1510-1842;
// the hwloc tree becomes the driver's P2P attribute matrix here).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace b200net {

enum class LinkType : uint8_t { SELF, NVLINK, PCIE, NONE };

// One PCI device on the way from the root complex to a GPU (a bridge or switch port).
struct TopoPciHop {
  std::string bus_id;       // "0000:17:00.0"
  std::string link_speed;   // sysfs current_link_speed, e.g. "32.0 GT/s PCIe" ("" when unknown)
  int link_width = 0;       // sysfs current_link_width
};

struct TopoGpu {
  int ordinal = 0;
  std::string pci_bus_id;   // "0000:1b:00.0"
  std::string name;
  int numa_node = -1;
  int cc_major = 0, cc_minor = 0;
  int sm_count = 0;
  bool multicast = false;   // NVSwitch multicast objects supported
  uint8_t uuid[16] = {0};
  // From sysfs: the bridges above the GPU, root first (empty in a VM that puts the GPU directly on
  // the root bus), and the GPU's own link.
  std::vector<TopoPciHop> pci_path;
  std::string link_speed;
  int link_width = 0;
};

struct TopoGroup {          // one GPU and the rails serving it
  int gpu;
  std::vector<int> rails;   // rail ids, ordered by the platform's sort_rails
  int speed_mbps;           // aggregate speed advertised for the group
};

class Topology {
 public:
  // Discover through the CUDA driver. Empty (no GPUs) when no driver is present.
  static Topology discover();
  // Fills numa_node, the link and the chain of bridges of `gpu` from <sysfs_root>/bus/pci/devices
  // (sysfs_root is "/sys" outside tests). False when the device is not there
  // (reference: the hwloc walk of src/nccl_ofi_topo.cpp:859-1259 and the link speed / width it
  // reads from sysfs, :1312-1498).
  static bool read_pci(TopoGpu* gpu, const std::string& sysfs_root = "/sys");
  // Build from a description (tests, tools): `links[i][j]` for every GPU pair.
  static Topology from_description(std::vector<TopoGpu> gpus, std::vector<std::vector<LinkType>> links);

  int num_gpus() const { return static_cast<int>(gpus_.size()); }
  const TopoGpu& gpu(int i) const { return gpus_[i]; }
  LinkType link(int a, int b) const { return links_[a][b]; }
  bool all_nvlink() const;           // every GPU pair connected by NVLink (an NVSwitch domain)
  bool nvls_capable() const;         // all_nvlink and every GPU supports multicast
  // Group rails with GPUs: every GPU gets `rails_per_gpu` copy channels.
  std::vector<TopoGroup> group(int rails_per_gpu, int rail_speed_mbps) const;
  // NCCL topology XML with one virtual NIC per GPU (speed scaled by the group size).
  std::string to_nccl_xml(const std::vector<TopoGroup>& groups) const;
  // Write the XML to an anonymous in-memory file and return a /proc/self/fd path for NCCL_TOPO_FILE
  // (the descriptor stays open for the life of the process). "" on failure.
  static std::string write_topo_memfd(const std::string& xml);

 private:
  std::vector<TopoGpu> gpus_;
  std::vector<std::vector<LinkType>> links_;
};

}  // namespace b200net
