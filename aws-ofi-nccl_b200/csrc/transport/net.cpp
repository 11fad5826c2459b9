// Plugin bring-up: parameters, CUDA driver, topology, platform selection, protocol selection,
// device creation, environment publication; plus the domain and endpoint caches
// (reference: src/nccl_ofi_net.cpp — create_plugin :179-421, properties :504-639, caches :706-940).
#include <limits.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <cstdio>

#include "b200net/cuda_shim.h"
#include "b200net/environ.h"
#include "b200net/log.h"
#include "b200net/net.h"
#include "b200net/param.h"
#include "b200net/plugin_stats.h"
#include "b200net/scheduler.h"
#include "b200net/shm_fabric.h"
#include "b200net/platform.h"
#include "b200net/system.h"
#include "b200net/topology.h"

extern char** environ;

namespace b200net {

// NVLink 5: 18 links x 50 GB/s per direction = 900 GB/s = 7.2 Tb/s per GPU.
constexpr int NVLINK5_GPU_MBPS = 7200000;
constexpr int HOST_PATH_MBPS = 200000;  // host-memory path (shared memory / cross-memory attach)

static std::mutex g_plugin_mu;
static Plugin* g_plugin = nullptr;
static int g_plugin_refs = 0;
static Topology* g_topo = nullptr;

Plugin* net_plugin() { return g_plugin; }

// ---------------------------------------------------------------- Domain / Device caches
Domain::Domain(Device* d) : device(d), mr_keys(size_t{1} << 16) {
  if (!params().mr_cache_disable.get()) mr_cache = std::make_unique<MrCache>(128);
}
Domain::~Domain() = default;

std::shared_ptr<Endpoint> Domain::get_ep() {
  std::lock_guard<std::mutex> g(lock);
  const long tid = current_tid();
  // purge entries whose endpoint is gone (their thread finished with it)
  for (auto it = ep_table_.begin(); it != ep_table_.end();) it = it->second.expired() ? ep_table_.erase(it) : std::next(it);
  auto it = ep_table_.find(tid);
  if (it != ep_table_.end()) {
    if (auto ep = it->second.lock()) {
      if (ep->is_active()) return ep;
      ep_table_.erase(it);  // an aborted endpoint is never handed out again
    }
  }
  std::shared_ptr<Endpoint> ep = create_endpoint();
  ep->domain_ref = shared_from_this();
  ep_table_[tid] = ep;
  return ep;
}

std::shared_ptr<Domain> Device::get_domain() {
  std::lock_guard<std::mutex> g(lock_);
  if (auto d = domain_.lock()) return d;
  std::shared_ptr<Domain> d = create_domain();
  domain_ = d;
  return d;
}

// ---------------------------------------------------------------- properties
static std::string pci_path_of_gpu(const std::string& bus_id) {
  if (bus_id.empty()) return "";
  std::string id = bus_id;
  for (auto& c : id) c = static_cast<char>(tolower(c));
  const std::string link = "/sys/bus/pci/devices/" + id;
  char buf[PATH_MAX];  // realpath() requires a PATH_MAX buffer
  if (!realpath(link.c_str(), buf)) return "";
  // Report the bridge above the GPU: NCCL then places the virtual NIC as a sibling of the GPU
  // under the same switch. Without a bridge above (GPU directly on a root port) report nothing and
  // let NCCL attach the NIC to the CPU.
  std::string path(buf);
  const size_t slash = path.rfind('/');
  if (slash == std::string::npos) return "";
  const std::string parent = path.substr(0, slash);
  const std::string leaf = parent.substr(parent.rfind('/') + 1);
  if (leaf.find(':') == std::string::npos || leaf.find('.') == std::string::npos) return "";
  return parent;
}

int fill_common_properties(Device* d, Properties* p, int rails) {
  if (!d || !p) return -EINVAL;
  Platform* plat = PlatformManager::instance().get_platform();
  p->name = d->name;
  p->guid = plat ? plat->device_get_guid(d->dev_id) : static_cast<uint64_t>(d->dev_id);
  p->latency_us = plat ? plat->latency_us() : 0.f;
  p->port = 1;
  p->force_flush = 0;
  p->max_comms = NET_MAX_COMMS;
  p->max_multi_request_size = 1;
  p->rail_id = -1;
  p->plane_id = -1;
  p->ptr_support = NCCL_PTR_HOST;
  p->port_speed_mbps = HOST_PATH_MBPS;
  if (d->gpu_ordinal >= 0 && g_topo && d->gpu_ordinal < g_topo->num_gpus()) {
    p->ptr_support |= NCCL_PTR_CUDA;
    if (!params().disable_dmabuf.get() && !params().nccl_device_buffers.get() && cuda::dmabuf_supported(d->gpu_ordinal))
      p->ptr_support |= NCCL_PTR_DMABUF;
    p->pci_path = pci_path_of_gpu(g_topo->gpu(d->gpu_ordinal).pci_bus_id);
    p->port_speed_mbps = g_topo->all_nvlink() ? NVLINK5_GPU_MBPS : 256000;  // PCIe gen5 x16 otherwise
  }
  (void)rails;
  return 0;
}

// ---------------------------------------------------------------- plugin creation
int net_create_plugin(Plugin** out) {
  std::lock_guard<std::mutex> g(g_plugin_mu);
  if (g_plugin) {
    ++g_plugin_refs;
    if (out) *out = g_plugin;
    return 0;
  }
  if (parameters_init() != 0) return -EINVAL;
  const int stale = FabricEndpoint::collect_stale_segments();
  if (stale) NET_INFO(NCCL_INIT, "removed %d shared-memory segment(s) of processes that no longer exist", stale);
  cuda::init();  // optional: without a driver only host buffers are served
  auto* topo = new Topology(Topology::discover());
  PlatformManager& pm = PlatformManager::instance();
  pm.register_all_platforms();
  Platform* plat = pm.get_platform();
  std::string provider_filter;
  if (plat && plat->init(&provider_filter) != 0) {
    delete topo;
    return -EINVAL;
  }

  // rails = stripes a large message is cut into: forced, else 1. One copy-kernel launch with
  // enough CTAs moves a whole message; more rails only add launches on the same stream.
  int rails = params().force_num_rails.get();
  if (rails <= 0) rails = 1;
  if (rails > MAX_NUM_RAILS) rails = MAX_NUM_RAILS;

  // protocol: parameter, then platform default, then by rail count
  std::string proto = params().protocol.get();
  for (auto& c : proto) c = static_cast<char>(toupper(c));
  if (proto.empty() && plat && *plat->default_protocol()) proto = plat->default_protocol();
  if (proto.empty()) proto = rails > 1 ? "RDMA" : "SENDRECV";

  const int ndev = topo->num_gpus() > 0 ? topo->num_gpus() : 1;
  auto* p = new Plugin();
  int rc = (proto == "SENDRECV") ? sendrecv_create_devices(p, ndev) : rdma_create_devices(p, ndev, rails);
  if (rc != 0) {
    delete p;
    delete topo;
    return rc;
  }
  g_topo = topo;
  NET_INFO(NCCL_INIT | NCCL_NET, "plugin up: protocol %s, %d device(s), %d rail(s), platform %s, NVSwitch %s, NVLS %s",
           p->protocol.c_str(), ndev, rails, plat ? plat->get_name() : "?", topo->all_nvlink() ? "yes" : "no",
           topo->nvls_capable() ? "yes" : "no");

  // Optionally give NCCL a topology file that puts net device i next to GPU i. Off by default:
  // the PCI path reported in the properties (the GPU's own) already places each virtual NIC.
  if (topo->num_gpus() > 0 && !getenv("NCCL_TOPO_FILE") &&
      (params().nccl_topo_inject.get() || !params().topo_file_write.get().empty())) {
    const auto groups = topo->group(rails, NVLINK5_GPU_MBPS / rails);
    const std::string xml = topo->to_nccl_xml(groups);
    const std::string path = Topology::write_topo_memfd(xml);
    if (!path.empty() && params().nccl_topo_inject.get())
      EnvManager::instance().insert_envvar("NCCL_TOPO_FILE", path, false);
    const std::string copy = params().topo_file_write.get();
    if (!copy.empty()) {
      if (FILE* f = fopen(copy.c_str(), "w")) {
        fputs(xml.c_str(), f);
        fclose(f);
      }
    }
  }
  // without device-memory support NCCL must not use the LL128 protocol through host bounce buffers
  if (topo->num_gpus() == 0) EnvManager::instance().insert_envvar("NCCL_PROTO", "simple", false);
  EnvManager::instance().update_environment(&environ);

  g_plugin = p;
  g_plugin_refs = 1;
  if (out) *out = p;
  return 0;
}

void net_destroy_plugin() {
  std::lock_guard<std::mutex> g(g_plugin_mu);
  if (!g_plugin || --g_plugin_refs > 0) return;
  HostCopyPool::instance().shutdown();   // no thread of this library outlives the plugin
  delete g_plugin;
  g_plugin = nullptr;
  delete g_topo;
  g_topo = nullptr;
}

void Endpoint::invalidate() {
  if (active.exchange(false)) PluginStats::bump(PluginStats::get().endpoints_aborted);
}

}  // namespace b200net
