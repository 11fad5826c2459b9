#include "b200net/topology.h"

#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstring>
#include <cstdio>

#include "b200net/cuda_shim.h"
#include "b200net/log.h"
#include "b200net/platform.h"

namespace b200net {

static int read_numa_node(const std::string& bus_id) {
  std::string id = bus_id;
  std::transform(id.begin(), id.end(), id.begin(), [](unsigned char c) { return std::tolower(c); });
  int n = -1;
  if (FILE* f = fopen(("/sys/bus/pci/devices/" + id + "/numa_node").c_str(), "r")) {
    if (fscanf(f, "%d", &n) != 1) n = -1;
    fclose(f);
  }
  return n;
}

Topology Topology::discover() {
  Topology t;
  const int n = cuda::device_count();
  for (int i = 0; i < n; ++i) {
    TopoGpu g;
    g.ordinal = i;
    char bus[32] = {0};
    if (cuda::device_pci_bus_id(i, bus, sizeof(bus)) == 0) g.pci_bus_id = bus;
    g.numa_node = read_numa_node(g.pci_bus_id);
    cuda::device_attribute(75, i, &g.cc_major);   // COMPUTE_CAPABILITY_MAJOR
    cuda::device_attribute(76, i, &g.cc_minor);   // COMPUTE_CAPABILITY_MINOR
    cuda::device_attribute(16, i, &g.sm_count);   // MULTIPROCESSOR_COUNT
    int mc = 0;
    cuda::device_attribute(132, i, &mc);          // MULTICAST_SUPPORTED
    g.multicast = mc != 0;
    cuda::device_uuid(i, g.uuid);
    t.gpus_.push_back(g);
  }
  t.links_.assign(n, std::vector<LinkType>(n, LinkType::NONE));
  for (int a = 0; a < n; ++a) {
    for (int b = 0; b < n; ++b) {
      if (a == b) {
        t.links_[a][b] = LinkType::SELF;
        continue;
      }
      int access = 0, atomics = 0;
      cuda::p2p_attribute(2 /* ACCESS_SUPPORTED */, a, b, &access);
      cuda::p2p_attribute(3 /* NATIVE_ATOMIC_SUPPORTED */, a, b, &atomics);
      // native atomics between peers exist over NVLink, not over PCIe
      t.links_[a][b] = !access ? LinkType::NONE : atomics ? LinkType::NVLINK : LinkType::PCIE;
    }
  }
  return t;
}

Topology Topology::from_description(std::vector<TopoGpu> gpus, std::vector<std::vector<LinkType>> links) {
  Topology t;
  t.gpus_ = std::move(gpus);
  t.links_ = std::move(links);
  return t;
}

bool Topology::all_nvlink() const {
  if (gpus_.size() < 2) return false;
  for (size_t a = 0; a < gpus_.size(); ++a)
    for (size_t b = 0; b < gpus_.size(); ++b)
      if (a != b && links_[a][b] != LinkType::NVLINK) return false;
  return true;
}

bool Topology::nvls_capable() const {
  if (!all_nvlink()) return false;
  return std::all_of(gpus_.begin(), gpus_.end(), [](const TopoGpu& g) { return g.multicast; });
}

std::vector<TopoGroup> Topology::group(int rails_per_gpu, int rail_speed_mbps) const {
  std::vector<TopoGroup> out;
  Platform* plat = PlatformManager::instance().get_platform();
  for (const TopoGpu& g : gpus_) {
    TopoGroup grp;
    grp.gpu = g.ordinal;
    for (int r = 0; r < rails_per_gpu; ++r) grp.rails.push_back(g.ordinal * rails_per_gpu + r);
    if (plat) plat->sort_rails(grp.rails);
    grp.speed_mbps = rail_speed_mbps * rails_per_gpu;
    out.push_back(std::move(grp));
  }
  return out;
}

// <system version="1"><cpu numaid=..><pci busid=.. class="0x060400"><pci busid=GPU class="0x030200"/>
//   <pci busid=virtual class="0x020000"><nic><net name=.. dev=.. speed=.. port="0" guid=.. maxconn=.. gdr="1"/></nic></pci>
// </pci></cpu></system> — the GPU and its virtual NIC share a (virtual) switch, so NCCL's search
// pairs them with the shortest path.
std::string Topology::to_nccl_xml(const std::vector<TopoGroup>& groups) const {
  std::string o = "<system version=\"1\">\n";
  char line[512];
  std::vector<int> numas;
  for (const auto& g : gpus_) {
    const int n = g.numa_node < 0 ? 0 : g.numa_node;
    if (std::find(numas.begin(), numas.end(), n) == numas.end()) numas.push_back(n);
  }
  std::sort(numas.begin(), numas.end());
  if (numas.empty()) numas.push_back(0);
  for (int numa : numas) {
    snprintf(line, sizeof(line),
             "  <cpu numaid=\"%d\" affinity=\"\" arch=\"x86_64\" vendor=\"\" familyid=\"0\" modelid=\"0\">\n", numa);
    o += line;
    for (const auto& grp : groups) {
      const TopoGpu& g = gpus_[grp.gpu];
      if ((g.numa_node < 0 ? 0 : g.numa_node) != numa) continue;
      snprintf(line, sizeof(line),
               "    <pci busid=\"ffff:%02x:00.0\" class=\"0x060400\" link_speed=\"32.0 GT/s PCIe\" link_width=\"16\">\n",
               g.ordinal);
      o += line;
      snprintf(line, sizeof(line),
               "      <pci busid=\"%s\" class=\"0x030200\" link_speed=\"32.0 GT/s PCIe\" link_width=\"16\"/>\n",
               g.pci_bus_id.empty() ? "0000:00:00.0" : g.pci_bus_id.c_str());
      o += line;
      snprintf(line, sizeof(line),
               "      <pci busid=\"ffff:%02x:01.0\" class=\"0x020000\" link_speed=\"32.0 GT/s PCIe\" link_width=\"16\">\n",
               g.ordinal);
      o += line;
      o += "        <nic>\n";
      snprintf(line, sizeof(line),
               "          <net name=\"nvl%d\" dev=\"%d\" speed=\"%d\" port=\"0\" guid=\"0x%llx\" maxconn=\"32768\" gdr=\"1\"/>\n",
               g.ordinal, g.ordinal, grp.speed_mbps, 0xb200000000ull | static_cast<unsigned>(g.ordinal));
      o += line;
      o += "        </nic>\n      </pci>\n    </pci>\n";
    }
    o += "  </cpu>\n";
  }
  o += "</system>\n";
  return o;
}

std::string Topology::write_topo_memfd(const std::string& xml) {
  const int fd = memfd_create("b200net-topo", 0);
  if (fd < 0) return "";
  size_t off = 0;
  while (off < xml.size()) {
    const ssize_t n = write(fd, xml.data() + off, xml.size() - off);
    if (n <= 0) {
      close(fd);
      return "";
    }
    off += static_cast<size_t>(n);
  }
  return "/proc/self/fd/" + std::to_string(fd);
}

}  // namespace b200net
