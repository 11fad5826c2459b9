#include "b200net/platform.h"

#include <algorithm>

#include <dlfcn.h>
#include <limits.h>

#include <cerrno>
#include <cstdlib>
#include <cstring>

#include "b200net/cuda_shim.h"
#include "b200net/environ.h"
#include "b200net/log.h"
#include "b200net/param.h"
#include "b200net/system.h"

namespace b200net {

std::string Platform::register_tuner() const {
  if (!params().tuner_self_register.get() || getenv("NCCL_TUNER_PLUGIN")) return "";
  Dl_info info;
  static const int anchor = 0;   // any address inside this shared object
  if (!dladdr(&anchor, &info) || !info.dli_fname || !*info.dli_fname) return "";
  char resolved[PATH_MAX];
  const std::string path = realpath(info.dli_fname, resolved) ? resolved : info.dli_fname;
  // only a shared object can be named; a test program that links the code statically has no tuner to offer
  if (path.size() < 3 || path.find(".so") == std::string::npos) return "";
  EnvManager::instance().insert_envvar("NCCL_TUNER_PLUGIN", path, false);
  return path;
}

uint64_t Platform::device_get_guid(int dev_index) const {
  return (static_cast<uint64_t>(system_node_id()) << 8) | static_cast<uint64_t>(dev_index & 0xff);
}

// ---------------------------------------------------------------- B200
int PlatformB200::init(std::string*) {
  for (auto& [k, v] : nccl_env()) EnvManager::instance().insert_envvar(k, v, false);
  const std::string tuner = register_tuner();
  if (!tuner.empty()) NET_INFO(NCCL_INIT | NCCL_TUNING, "NCCL_TUNER_PLUGIN set to %s", tuner.c_str());
  return 0;
}

std::vector<std::pair<std::string, std::string>> PlatformB200::nccl_env() const {
  // Chunks sized for MiB-sized copies over NVLink rather than for NIC MTUs. NCCL attaches this
  // transport's virtual NICs to the CPU (they are no PCI devices), which is farther from the GPUs
  // than its default limit for handing device buffers to a network, so the limit is raised: the
  // "NIC" is the GPU's own NVLink port. LL128 stays off: it relies on a network that delivers the
  // bytes of a 128-byte line in order, which a copy kernel with many threads does not promise.
  std::vector<std::pair<std::string, std::string>> env = {{"NCCL_BUFFSIZE", "33554432"},
                                                          {"NCCL_P2P_NET_CHUNKSIZE", "4194304"},
                                                          {"NCCL_NVLS_CHUNKSIZE", "524288"},
                                                          {"NCCL_NET_FORCE_FLUSH", "0"},
                                                          {"NCCL_PROTO", "^LL128"},
                                                          // sixteen channels are connected; the tuner gives each call as
                                                          // many of them as its size is worth
                                                          {"NCCL_MIN_NCHANNELS", "16"}};
  // NCCL_NCHANNELS_PER_NET_PEER (channels per peer for point-to-point calls; 8 instead of NCCL's 2
  // took a 256 MiB all_to_all on two B200 from 45 to 166 GB/s) cannot be set from here: NCCL reads
  // it before it initialises its net plugin. Launchers export it themselves.
  if (params().nccl_device_buffers.get()) {
    env.emplace_back("NCCL_NET_GDR_LEVEL", "SYS");
    env.emplace_back("NCCL_NET_GDR_READ", "1");
  }
  return env;
}

std::string PlatformB200::log_error_hint(int err) const {
  switch (err) {
    case EHOSTUNREACH:
      return "the peer's endpoint segment could not be opened: is /dev/shm shared between the ranks (same IPC namespace)?";
    case ENOTCONN:
      return "the peer closed its endpoint: a rank exited or tore down its communicator early";
    case EPERM:
      return "cross-memory attach was refused: set B200NET_DISABLE_CMA=1 or allow ptrace between the ranks";
    default:
      return "";
  }
}

void PlatformB200::sort_rails(std::vector<int>& rails) { std::sort(rails.begin(), rails.end()); }

// ---------------------------------------------------------------- cloud instance table
const std::vector<InstanceEntry>& instance_table() {
  static const std::vector<std::pair<std::string, std::string>> p5_env = {
      {"NCCL_BUFFSIZE", "8388608"}, {"NCCL_P2P_NET_CHUNKSIZE", "524288"}, {"NCCL_NVLS_CHUNKSIZE", "524288"},
      {"NCCL_NET_FORCE_FLUSH", "0"}};
  static const std::vector<InstanceEntry> table = {
      {"p3dn.24xlarge", nullptr, nullptr, false, 150.f, false, "SENDRECV", false, {}},
      {"p4d.24xlarge", nullptr, "p4d-24xl-topo.xml", false, 75.f, true, "RDMA", false, {}},
      {"p4de.24xlarge", nullptr, "p4de-24xl-topo.xml", false, 75.f, true, "RDMA", false, {}},
      {"p5.48xlarge", "^p5e?\\.(4|48)xlarge$", nullptr, false, 75.f, true, "RDMA", false, p5_env},
      {"p5en.48xlarge", nullptr, nullptr, false, 35.f, true, "RDMA", true, p5_env},
      {"p6-b200.48xlarge", "^p6e?-b200\\..*$", nullptr, false, 35.f, true, "RDMA", true, p5_env},
      {"p6-b300.48xlarge", "^p6-b300\\..*$", nullptr, false, 35.f, true, "RDMA", true, p5_env},
      {"g5.48xlarge", nullptr, "g5.48xl-topo.xml", true, 75.f, false, "SENDRECV", false, {}},
      {"trn1.32xlarge", "^trn[12]n?\\..*$", nullptr, false, 75.f, true, "RDMA", false, {}},
  };
  return table;
}

const InstanceEntry* find_instance(const std::string& product) {
  if (product.empty()) return nullptr;
  for (const auto& e : instance_table()) {
    if (e.regex) {
      if (std::regex_match(product, std::regex(e.regex))) return &e;
    } else if (product == e.name) {
      return &e;
    }
  }
  return nullptr;
}

std::vector<std::pair<std::string, std::string>> PlatformCloud::nccl_env() const {
  return e_ ? e_->env : std::vector<std::pair<std::string, std::string>>{};
}

// ---------------------------------------------------------------- manager
PlatformManager& PlatformManager::instance() {
  static PlatformManager* m = new PlatformManager();
  return *m;
}

void PlatformManager::register_platform(std::unique_ptr<Platform> p) {
  platforms_.push_back(std::move(p));
  chosen_ = nullptr;
}

void PlatformManager::clear_for_testing() {
  platforms_.clear();
  chosen_ = nullptr;
}

static bool detect_b200() {
  const std::string product = system_product_name();
  if (product.find("B200") != std::string::npos || product.find("b200") != std::string::npos) return true;
  if (!cuda::available()) return false;
  int major = 0;
  // compute capability 10.x = Blackwell data-centre parts
  if (cuda::device_attribute(75 /* COMPUTE_CAPABILITY_MAJOR */, 0, &major) == 0 && major == 10) return true;
  return false;
}

void PlatformManager::register_all_platforms() {
  if (!platforms_.empty()) return;
  register_platform(std::make_unique<PlatformDefault>());
  register_platform(std::make_unique<PlatformB200>(detect_b200()));
  register_platform(std::make_unique<PlatformCloud>(find_instance(system_product_name())));
}

Platform* PlatformManager::get_platform() {
  if (chosen_) return chosen_;
  const std::string forced = params().platform.get();
  Platform* best = nullptr;
  for (auto& p : platforms_) {
    if (!forced.empty()) {
      if (forced == p->get_name()) {
        best = p.get();
        break;
      }
      continue;
    }
    if (p->get_priority() < 0) continue;
    if (!best || p->get_priority() > best->get_priority()) best = p.get();
  }
  if (!best && !forced.empty()) NET_WARN("platform '%s' requested but not registered", forced.c_str());
  if (!best)
    for (auto& p : platforms_)
      if (p->get_priority() >= 0 && (!best || p->get_priority() > best->get_priority())) best = p.get();
  chosen_ = best;
  return chosen_;
}

}  // namespace b200net
