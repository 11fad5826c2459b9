#include "b200net/topology.h"

#include <limits.h>
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <cstdio>

#include "b200net/cuda_shim.h"
#include "b200net/log.h"
#include "b200net/platform.h"

namespace b200net {

static std::string read_line(const std::string& path) {
  std::string out;
  if (FILE* f = fopen(path.c_str(), "r")) {
    char buf[128];
    if (fgets(buf, sizeof(buf), f)) out = buf;
    fclose(f);
  }
  while (!out.empty() && (out.back() == '\n' || out.back() == ' ')) out.pop_back();
  return out;
}

static bool looks_like_bdf(const std::string& s) {   // dddd:bb:dd.f
  return s.size() >= 12 && s[4] == ':' && s[7] == ':' && s[10] == '.';
}

bool Topology::read_pci(TopoGpu* gpu, const std::string& sysfs_root) {
  std::string id = gpu->pci_bus_id;
  std::transform(id.begin(), id.end(), id.begin(), [](unsigned char c) { return std::tolower(c); });
  if (id.empty()) return false;
  const std::string link = sysfs_root + "/bus/pci/devices/" + id;
  char real[PATH_MAX];
  if (!realpath(link.c_str(), real)) return false;
  const std::string numa = read_line(link + "/numa_node");
  gpu->numa_node = numa.empty() ? -1 : atoi(numa.c_str());
  gpu->link_speed = read_line(link + "/current_link_speed");
  gpu->link_width = atoi(read_line(link + "/current_link_width").c_str());
  // /sys/devices/pci0000:15/0000:15:01.0/0000:16:00.0/0000:17:00.0/<gpu>: every component that is a
  // bus address, except the last, is a bridge above the GPU
  gpu->pci_path.clear();
  std::string path(real), built;
  size_t pos = 0;
  std::vector<std::string> parts;
  while (pos <= path.size()) {
    const size_t next = path.find('/', pos);
    parts.push_back(path.substr(pos, next == std::string::npos ? std::string::npos : next - pos));
    if (next == std::string::npos) break;
    pos = next + 1;
  }
  for (size_t i = 0; i < parts.size(); ++i) {
    built += (i ? "/" : "") + parts[i];
    if (i + 1 == parts.size() || !looks_like_bdf(parts[i])) continue;
    TopoPciHop hop;
    hop.bus_id = parts[i];
    hop.link_speed = read_line(built + "/current_link_speed");
    hop.link_width = atoi(read_line(built + "/current_link_width").c_str());
    gpu->pci_path.push_back(hop);
  }
  return true;
}

Topology Topology::discover() {
  Topology t;
  const int n = cuda::device_count();
  for (int i = 0; i < n; ++i) {
    TopoGpu g;
    g.ordinal = i;
    char bus[32] = {0};
    if (cuda::device_pci_bus_id(i, bus, sizeof(bus)) == 0) g.pci_bus_id = bus;
    read_pci(&g);
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
    // GPUs of this NUMA node as a tree of the bridges above them (GPUs behind one switch share its
    // node); a GPU with no bridge above it gets a virtual one, so that it and its NIC have a
    // common parent below the CPU and NCCL's search pairs them with the shortest path
    std::vector<std::string> open_path;   // bridges currently open in the output
    auto close_to = [&](size_t depth) {
      while (open_path.size() > depth) {
        o += std::string(2 + 2 * open_path.size(), ' ') + "</pci>\n";
        open_path.pop_back();
      }
    };
    std::vector<const TopoGroup*> here;
    for (const auto& grp : groups)
      if ((gpus_[grp.gpu].numa_node < 0 ? 0 : gpus_[grp.gpu].numa_node) == numa) here.push_back(&grp);
    auto path_key = [&](const TopoGroup* grp) {
      std::string k;
      for (const TopoPciHop& h : gpus_[grp->gpu].pci_path) k += h.bus_id + "/";
      return k;
    };
    std::stable_sort(here.begin(), here.end(), [&](const TopoGroup* a, const TopoGroup* b) { return path_key(a) < path_key(b); });
    for (const TopoGroup* grp_p : here) {
      const TopoGroup& grp = *grp_p;
      const TopoGpu& g = gpus_[grp.gpu];
      std::vector<TopoPciHop> path = g.pci_path;
      if (path.empty()) {
        TopoPciHop v;
        char id[32];
        snprintf(id, sizeof(id), "ffff:%02x:00.0", g.ordinal);
        v.bus_id = id;
        v.link_speed = "32.0 GT/s PCIe";
        v.link_width = 16;
        path.push_back(v);
      }
      size_t common = 0;
      while (common < open_path.size() && common < path.size() && open_path[common] == path[common].bus_id) ++common;
      close_to(common);
      for (size_t d = common; d < path.size(); ++d) {
        snprintf(line, sizeof(line), "%*s<pci busid=\"%s\" class=\"0x060400\" link_speed=\"%s\" link_width=\"%d\">\n",
                 static_cast<int>(4 + 2 * d), "", path[d].bus_id.c_str(),
                 path[d].link_speed.empty() ? "32.0 GT/s PCIe" : path[d].link_speed.c_str(), path[d].link_width ? path[d].link_width : 16);
        o += line;
        open_path.push_back(path[d].bus_id);
      }
      const int ind = static_cast<int>(4 + 2 * path.size());
      snprintf(line, sizeof(line), "%*s<pci busid=\"%s\" class=\"0x030200\" link_speed=\"%s\" link_width=\"%d\"/>\n", ind, "",
               g.pci_bus_id.empty() ? "0000:00:00.0" : g.pci_bus_id.c_str(), g.link_speed.empty() ? "32.0 GT/s PCIe" : g.link_speed.c_str(),
               g.link_width ? g.link_width : 16);
      o += line;
      snprintf(line, sizeof(line), "%*s<pci busid=\"ffff:%02x:01.0\" class=\"0x020000\" link_speed=\"32.0 GT/s PCIe\" link_width=\"16\">\n", ind, "",
               g.ordinal);
      o += line;
      snprintf(line, sizeof(line), "%*s<nic>\n", ind + 2, "");
      o += line;
      snprintf(line, sizeof(line),
               "%*s<net name=\"nvl%d\" dev=\"%d\" speed=\"%d\" port=\"0\" guid=\"0x%llx\" maxconn=\"32768\" gdr=\"1\"/>\n", ind + 4, "",
               g.ordinal, g.ordinal, grp.speed_mbps, 0xb200000000ull | static_cast<unsigned>(g.ordinal));
      o += line;
      snprintf(line, sizeof(line), "%*s</nic>\n%*s</pci>\n", ind + 2, "", ind, "");
      o += line;
    }
    close_to(0);
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
