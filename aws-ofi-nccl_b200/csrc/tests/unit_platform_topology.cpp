// Platform manager (priority selection with fake platforms, forcing by name), topology grouping and
// the generated NCCL topology XML, system helpers.
#include <algorithm>
#include <cstring>
#include <string>
#include "b200net/param.h"
#include "b200net/platform.h"
#include "b200net/system.h"
#include "b200net/topology.h"
#include "test_util.h"
using namespace b200net;

class FakePlatform : public Platform {
 public:
  FakePlatform(const char* n, int prio) : n_(n), p_(prio) {}
  const char* get_name() const override { return n_; }
  int get_priority() const override { return p_; }
  void sort_rails(std::vector<int>& rails) override { std::reverse(rails.begin(), rails.end()); }
 private:
  const char* n_; int p_;
};

int main() {
  PlatformManager& pm = PlatformManager::instance();
  pm.clear_for_testing();
  pm.register_platform(std::make_unique<PlatformDefault>());
  CHECK(!strcmp(pm.get_platform()->get_name(), "Default"));
  pm.register_platform(std::make_unique<FakePlatform>("Low", 10));
  pm.register_platform(std::make_unique<FakePlatform>("High", 90));
  pm.register_platform(std::make_unique<FakePlatform>("NotHere", -1));
  CHECK(!strcmp(pm.get_platform()->get_name(), "High"));
  pm.register_platform(std::make_unique<PlatformB200>(true));
  CHECK(!strcmp(pm.get_platform()->get_name(), "B200"));
  CHECK(pm.get_platform()->gdaki_capable());
  CHECK(!pm.get_platform()->log_error_hint(EHOSTUNREACH).empty());
  CHECK(pm.get_platform()->log_error_hint(0).empty());
  CHECK(pm.get_platform()->device_get_guid(3) != pm.get_platform()->device_get_guid(4));
  // forcing by name beats priority (parameter read happens inside get_platform)
  pm.clear_for_testing();
  params().platform.reset_for_testing("");
  params().platform.set("Low");
  pm.register_platform(std::make_unique<PlatformDefault>());
  pm.register_platform(std::make_unique<FakePlatform>("Low", 10));
  pm.register_platform(std::make_unique<FakePlatform>("High", 90));
  CHECK(!strcmp(pm.get_platform()->get_name(), "Low"));

  // ---- topology from a description: 4 GPUs on NVSwitch, 2 NUMA nodes
  std::vector<TopoGpu> gpus(4);
  for (int i = 0; i < 4; ++i) {
    gpus[i].ordinal = i;
    char b[32]; snprintf(b, sizeof(b), "0000:%02x:00.0", 0x10 + i * 0x10);
    gpus[i].pci_bus_id = b; gpus[i].numa_node = i / 2; gpus[i].multicast = true; gpus[i].cc_major = 10;
  }
  std::vector<std::vector<LinkType>> links(4, std::vector<LinkType>(4, LinkType::NVLINK));
  for (int i = 0; i < 4; ++i) links[i][i] = LinkType::SELF;
  Topology t = Topology::from_description(gpus, links);
  CHECK(t.all_nvlink() && t.nvls_capable());
  auto groups = t.group(4, 1800000);
  CHECK_EQ(groups.size(), 4u);
  CHECK_EQ(groups[2].rails.size(), 4u);
  CHECK_EQ(groups[2].rails[0], 11);          // the forced platform reverses rails: 8,9,10,11 -> 11..8
  CHECK_EQ(groups[2].speed_mbps, 7200000);
  const std::string xml = t.to_nccl_xml(groups);
  const char* golden_lines[] = {
      "<system version=\"1\">", "<cpu numaid=\"0\"", "<cpu numaid=\"1\"",
      "<pci busid=\"0000:10:00.0\" class=\"0x030200\"", "<pci busid=\"0000:40:00.0\" class=\"0x030200\"",
      "<net name=\"nvl0\" dev=\"0\" speed=\"7200000\" port=\"0\" guid=\"0xb200000000\" maxconn=\"32768\" gdr=\"1\"/>",
      "<net name=\"nvl3\" dev=\"3\" speed=\"7200000\"", "</system>"};
  for (const char* g : golden_lines) CHECK(xml.find(g) != std::string::npos);
  CHECK(xml.find("nvl0") < xml.find("nvl1") && xml.find("numaid=\"0\"") < xml.find("nvl1") && xml.find("nvl1") < xml.find("numaid=\"1\""));
  const std::string path = Topology::write_topo_memfd(xml);
  CHECK(!path.empty());
  FILE* f = fopen(path.c_str(), "r");
  CHECK(f != nullptr);
  if (f) { char head[32] = {0}; CHECK(fread(head, 1, 22, f) == 22); CHECK(!strncmp(head, "<system version=\"1\">", 20)); fclose(f); }
  links[0][3] = links[3][0] = LinkType::PCIE;
  CHECK(!Topology::from_description(gpus, links).all_nvlink());
  gpus[1].multicast = false;
  links[0][3] = links[3][0] = LinkType::NVLINK;
  CHECK(!Topology::from_description(gpus, links).nvls_capable());
  CHECK(!Topology::from_description({}, {}).all_nvlink());

  // ---- PCI hierarchy from a (fake) sysfs tree: two GPUs behind one switch, a third on a root port of its own
  {
    char tmpl[] = "/tmp/b200net-sysfs-XXXXXX";
    const std::string root = mkdtemp(tmpl);
    auto sh = [&](const std::string& cmd) { return system(cmd.c_str()); };
    const std::string dev = root + "/devices/pci0000:15";
    CHECK_EQ(sh("mkdir -p " + dev + "/0000:15:01.0/0000:16:00.0/0000:17:00.0/0000:18:00.0 " + dev + "/0000:15:01.0/0000:16:00.0/0000:17:01.0/0000:19:00.0 " +
                root + "/devices/pci0000:80/0000:80:01.0/0000:81:00.0 " + root + "/bus/pci/devices"), 0);
    for (const char* bdf : {"0000:15:01.0/0000:16:00.0/0000:17:00.0/0000:18:00.0", "0000:15:01.0/0000:16:00.0/0000:17:01.0/0000:19:00.0"}) {
      const std::string d = dev + "/" + bdf, leaf = d.substr(d.rfind('/') + 1);
      sh("echo 0 > " + d + "/numa_node; echo '32.0 GT/s PCIe' > " + d + "/current_link_speed; echo 16 > " + d + "/current_link_width");
      sh("ln -s " + d + " " + root + "/bus/pci/devices/" + leaf);
    }
    sh("echo '16.0 GT/s PCIe' > " + dev + "/0000:15:01.0/0000:16:00.0/current_link_speed; echo 8 > " + dev + "/0000:15:01.0/0000:16:00.0/current_link_width");
    const std::string d3 = root + "/devices/pci0000:80/0000:80:01.0/0000:81:00.0";
    sh("echo 1 > " + d3 + "/numa_node; ln -s " + d3 + " " + root + "/bus/pci/devices/0000:81:00.0");
    std::vector<TopoGpu> pg(3);
    const char* ids[] = {"0000:18:00.0", "0000:19:00.0", "0000:81:00.0"};
    for (int i = 0; i < 3; ++i) {
      pg[i].ordinal = i;
      pg[i].pci_bus_id = ids[i];
      CHECK(Topology::read_pci(&pg[i], root));
    }
    CHECK_EQ(pg[0].pci_path.size(), 3u);
    CHECK(pg[0].pci_path[0].bus_id == "0000:15:01.0" && pg[0].pci_path[2].bus_id == "0000:17:00.0");
    CHECK(pg[0].pci_path[1].link_speed == "16.0 GT/s PCIe" && pg[0].pci_path[1].link_width == 8);
    CHECK(pg[0].link_width == 16 && pg[0].numa_node == 0 && pg[2].numa_node == 1);
    CHECK_EQ(pg[2].pci_path.size(), 1u);
    TopoGpu missing;
    missing.pci_bus_id = "0000:ff:00.0";
    CHECK(!Topology::read_pci(&missing, root));
    std::vector<std::vector<LinkType>> l3(3, std::vector<LinkType>(3, LinkType::NVLINK));
    Topology pt = Topology::from_description(pg, l3);
    const std::string px = pt.to_nccl_xml(pt.group(1, 7200000));
    // the two GPUs behind the switch share its upstream bridges (each named once), then split at the switch ports
    CHECK(px.find("0000:16:00.0") != std::string::npos && px.find("0000:16:00.0") == px.rfind("0000:16:00.0"));
    CHECK(px.find("busid=\"0000:17:00.0\"") < px.find("busid=\"0000:18:00.0\"") && px.find("busid=\"0000:18:00.0\"") < px.find("nvl0"));
    CHECK(px.find("nvl0") < px.find("busid=\"0000:17:01.0\"") && px.find("busid=\"0000:17:01.0\"") < px.find("nvl1"));
    CHECK(px.find("link_speed=\"16.0 GT/s PCIe\" link_width=\"8\"") != std::string::npos);
    CHECK(px.find("numaid=\"1\"") < px.find("busid=\"0000:80:01.0\"") && px.find("busid=\"0000:80:01.0\"") < px.find("nvl2"));
    size_t opens = 0, closes = 0;
    for (size_t p2 = 0; (p2 = px.find("<pci ", p2)) != std::string::npos; ++p2) ++opens;
    for (size_t p2 = 0; (p2 = px.find("</pci>", p2)) != std::string::npos; ++p2) ++closes;
    size_t selfclosed = 0;
    for (size_t p2 = 0; (p2 = px.find("\"/>\n", p2)) != std::string::npos; ++p2) ++selfclosed;
    CHECK_EQ(opens, closes + 3u);   // the three GPU nodes are self-closing (the <net/> lines are not <pci>)
    (void)selfclosed;
    sh("rm -rf " + root);
  }

  // ---- system helpers
  setenv("OFI_NCCL_FORCE_PRODUCT_NAME", "p5en.48xlarge", 1);
  CHECK(system_product_name() == "p5en.48xlarge");
  unsetenv("OFI_NCCL_FORCE_PRODUCT_NAME");
  setenv("NCCL_HOSTID", "abc", 1);
  {
    PlatformB200 b200(true);
    std::vector<int> rails{3, 0, 2, 1};
    b200.sort_rails(rails);
    CHECK(rails == (std::vector<int>{0, 1, 2, 3}));   // both ends of a connection enumerate rails alike
  }
  const uint64_t h1 = system_host_hash();
  setenv("NCCL_HOSTID", "abd", 1);
  CHECK(h1 != system_host_hash());
  unsetenv("NCCL_HOSTID");
  CHECK(system_host_hash() == system_host_hash());
  CHECK(current_tid() > 0);
  TEST_MAIN_END();
}
