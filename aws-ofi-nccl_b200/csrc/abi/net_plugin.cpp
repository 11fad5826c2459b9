// Exported ncclNet tables, ABI versions 6 to 12. NCCL dlsym()s the newest "ncclNetPlugin_vN" it
// knows; each table adapts that generation's signatures and property struct to the validated API
// (reference: src/nccl_ofi_interface_nvidia.cpp:661-858).
#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <atomic>
#include <climits>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "b200net/api.h"
#include "b200net/log.h"
#include "b200net/param.h"

using namespace b200net;

#define B200NET_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

char g_name[64] = "B200NVL";

// NCCL only accepts a plugin whose name equals NCCL_NET when that variable is set: adopt the
// requested name at load time so that a forced selection still finds this plugin.
__attribute__((constructor)) void adopt_requested_name() {
  const char* want = getenv("NCCL_NET");
  if (want && *want && strcasecmp(want, "IB") != 0 && strcasecmp(want, "Socket") != 0)
    snprintf(g_name, sizeof(g_name), "%s", want);
}

// Debug aid: with B200NET_SEGV_BACKTRACE=1 a crash inside the process prints raw return addresses
// (resolve them against the .so with addr2line) before the default action runs.
void segv_backtrace(int sig) {
  void* frames[64];
  const int n = backtrace(frames, 64);
  const char msg[] = "\n[b200net] fatal signal, backtrace:\n";
  if (write(2, msg, sizeof(msg) - 1) < 0) {}
  backtrace_symbols_fd(frames, n, 2);
  signal(sig, SIG_DFL);
  raise(sig);
}
__attribute__((constructor)) void install_segv_backtrace() {
  const char* e = getenv("B200NET_SEGV_BACKTRACE");
  if (e && *e == '1') {
    signal(SIGSEGV, segv_backtrace);
    signal(SIGBUS, segv_backtrace);
    signal(SIGABRT, segv_backtrace);
  }
}

// The strings returned in property structs must outlive the call: keep one copy per device.
std::mutex g_props_mu;
struct PropStrings { std::string name, pci; };
PropStrings g_prop_strings[64];

ncclResult_t props_common(int dev, Properties* p, char** name, char** pci) {
  const ncclResult_t r = api::get_properties(dev, p);
  if (r != ncclSuccess) return r;
  std::lock_guard<std::mutex> g(g_props_mu);
  PropStrings& s = g_prop_strings[dev % 64];
  s.name = p->name;
  s.pci = p->pci_path;
  *name = const_cast<char*>(s.name.c_str());
  *pci = s.pci.empty() ? nullptr : const_cast<char*>(s.pci.c_str());
  return ncclSuccess;
}

template <typename P>
void fill_v6_fields(P* out, const Properties& p, char* name, char* pci, int max_recvs) {
  out->name = name;
  out->pciPath = pci;
  out->guid = p.guid;
  out->ptrSupport = p.ptr_support;
  out->speed = p.port_speed_mbps;
  out->port = p.port;
  out->latency = p.latency_us;
  out->maxComms = p.max_comms;
  out->maxRecvs = max_recvs;
}

// ---- init / finalize bookkeeping --------------------------------------------------------------
std::mutex g_init_mu;
int g_init_refs = 0;
std::atomic<int> g_traffic_class{-1};
bool g_atexit_registered = false;

void fini_at_exit() {
  std::lock_guard<std::mutex> g(g_init_mu);
  while (g_init_refs > 0) {
    api::fini();
    --g_init_refs;
  }
}

ncclResult_t init_common(ncclDebugLogger_t log_fn, bool legacy) {
  std::lock_guard<std::mutex> g(g_init_mu);
  const ncclResult_t r = api::init(log_fn);
  if (r != ncclSuccess) return r;
  ++g_init_refs;
  // ABIs before v11 have no finalize(): release everything when the process exits
  if (legacy && !g_atexit_registered) {
    atexit(fini_at_exit);
    g_atexit_registered = true;
  }
  return ncclSuccess;
}

ncclResult_t init_v6(ncclDebugLogger_t log_fn) { return init_common(log_fn, true); }
// NCCL's profiler callback is accepted and not used.
ncclResult_t init_v10(ncclDebugLogger_t log_fn, ncclProfilerCallback_t) { return init_common(log_fn, true); }
ncclResult_t init_v11(void** ctx, uint64_t, ncclNetCommConfig_t* config, ncclDebugLogger_t log_fn, ncclProfilerCallback_t) {
  if (config) g_traffic_class.store(config->trafficClass);
  const ncclResult_t r = init_common(log_fn, false);
  if (ctx) *ctx = r == ncclSuccess ? reinterpret_cast<void*>(&g_init_refs) : nullptr;
  return r;
}
ncclResult_t finalize_v11(void*) {
  std::lock_guard<std::mutex> g(g_init_mu);
  if (g_init_refs <= 0) return ncclInvalidUsage;
  --g_init_refs;
  return api::fini();
}

ncclResult_t devices(int* n) { return api::devices(n); }

// ---- properties per generation --------------------------------------------------------------------
ncclResult_t get_properties_v6(int dev, ncclNetProperties_v6_t* out) {
  if (!out) return ncclInvalidArgument;
  Properties p;
  char *name, *pci;
  const ncclResult_t r = props_common(dev, &p, &name, &pci);
  if (r != ncclSuccess) return r;
  fill_v6_fields(out, p, name, pci, 1);  // grouped receives need the v9+ size_t interfaces
  return ncclSuccess;
}
ncclResult_t get_properties_v7(int dev, ncclNetProperties_v7_t* out) {
  if (!out) return ncclInvalidArgument;
  Properties p;
  char *name, *pci;
  const ncclResult_t r = props_common(dev, &p, &name, &pci);
  if (r != ncclSuccess) return r;
  fill_v6_fields(out, p, name, pci, 1);
  out->netDeviceType = NCCL_NET_DEVICE_HOST;
  out->netDeviceVersion = NCCL_NET_DEVICE_INVALID_VERSION;
  return ncclSuccess;
}
ncclResult_t get_properties_v8(int dev, ncclNetProperties_v8_t* out) {
  if (!out) return ncclInvalidArgument;
  Properties p;
  char *name, *pci;
  const ncclResult_t r = props_common(dev, &p, &name, &pci);
  if (r != ncclSuccess) return r;
  fill_v6_fields(out, p, name, pci, 1);
  out->regIsGlobal = p.reg_is_global;
  out->netDeviceType = NCCL_NET_DEVICE_HOST;
  out->netDeviceVersion = NCCL_NET_DEVICE_INVALID_VERSION;
  return ncclSuccess;
}
template <typename P>
ncclResult_t get_properties_v9plus(int dev, P* out) {
  if (!out) return ncclInvalidArgument;
  Properties p;
  char *name, *pci;
  const ncclResult_t r = props_common(dev, &p, &name, &pci);
  if (r != ncclSuccess) return r;
  fill_v6_fields(out, p, name, pci, p.max_recvs);
  out->regIsGlobal = p.reg_is_global;
  out->forceFlush = p.force_flush;
  out->netDeviceType = NCCL_NET_DEVICE_HOST;
  out->netDeviceVersion = NCCL_NET_DEVICE_INVALID_VERSION;
  out->vProps.ndevs = 1;
  out->vProps.devs[0] = dev;
  out->maxP2pBytes = p.max_p2p_bytes;
  out->maxCollBytes = p.max_coll_bytes;
  return ncclSuccess;
}
ncclResult_t get_properties_v9(int dev, ncclNetProperties_v9_t* out) { return get_properties_v9plus(dev, out); }
ncclResult_t get_properties_v11(int dev, ncclNetProperties_v11_t* out) {
  const ncclResult_t r = get_properties_v9plus(dev, out);
  if (r == ncclSuccess) out->maxMultiRequestSize = 1;
  return r;
}
ncclResult_t get_properties_v12(int dev, ncclNetProperties_v12_t* out) {
  const ncclResult_t r = get_properties_v9plus(dev, out);
  if (r == ncclSuccess) {
    out->maxMultiRequestSize = 1;
    out->railId = -1;
    out->planeId = -1;
  }
  return r;
}

// ---- connection calls ------------------------------------------------------------------------------
ncclResult_t listen_v6(int dev, void* handle, void** l) { return api::listen(dev, handle, l); }
ncclResult_t listen_v11(void*, int dev, void* handle, void** l) { return api::listen(dev, handle, l); }
ncclResult_t connect_v6(int dev, void* handle, void** s) { return api::connect(dev, handle, s, -1); }
ncclResult_t connect_v7(int dev, void* handle, void** s, ncclNetDeviceHandle_t** dh) {
  if (dh) *dh = nullptr;
  return api::connect(dev, handle, s, -1);
}
ncclResult_t connect_v10(int dev, ncclNetCommConfig_t* cfg, void* handle, void** s, ncclNetDeviceHandle_t** dh) {
  if (dh) *dh = nullptr;
  return api::connect(dev, handle, s, cfg ? cfg->trafficClass : -1);
}
ncclResult_t connect_v11(void*, int dev, void* handle, void** s, ncclNetDeviceHandle_t** dh) {
  if (dh) *dh = nullptr;
  return api::connect(dev, handle, s, g_traffic_class.load());
}
ncclResult_t accept_v6(void* l, void** r) { return api::accept(l, r); }
ncclResult_t accept_v7(void* l, void** r, ncclNetDeviceHandle_t** dh) {
  if (dh) *dh = nullptr;
  return api::accept(l, r);
}

// ---- memory registration ---------------------------------------------------------------------------
ncclResult_t reg_mr_v6(void* c, void* d, int size, int type, void** mh) {
  if (size < 0) return ncclInvalidArgument;
  return api::reg_mr(c, d, static_cast<size_t>(size), type, mh);
}
ncclResult_t reg_mr_v8(void* c, void* d, size_t size, int type, void** mh) { return api::reg_mr(c, d, size, type, mh); }
ncclResult_t reg_mr_dmabuf(void* c, void* d, size_t size, int type, uint64_t off, int fd, void** mh) {
  return api::reg_mr_dmabuf(c, d, size, type, off, fd, mh);
}
ncclResult_t dereg_mr(void* c, void* mh) { return api::dereg_mr(c, mh); }

// ---- data calls ------------------------------------------------------------------------------------
ncclResult_t isend_v6(void* s, void* d, int size, int tag, void* mh, void** req) {
  if (size < 0) return ncclInvalidArgument;
  return api::isend(s, d, static_cast<size_t>(size), tag, mh, req);
}
ncclResult_t isend_v9(void* s, void* d, size_t size, int tag, void* mh, void** req) {
  return api::isend(s, d, size, tag, mh, req);
}
ncclResult_t isend_v10(void* s, void* d, size_t size, int tag, void* mh, void*, void** req) {
  return api::isend(s, d, size, tag, mh, req);
}
ncclResult_t irecv_v6(void* r, int n, void** d, int* sizes, int* tags, void** mh, void** req) {
  if (n < 1 || n > NET_MAX_RECVS || !sizes) return ncclInvalidArgument;
  size_t s64[NET_MAX_RECVS];
  for (int i = 0; i < n; ++i) {
    if (sizes[i] < 0) return ncclInvalidArgument;
    s64[i] = static_cast<size_t>(sizes[i]);
  }
  return api::irecv(r, n, d, s64, tags, mh, req);
}
ncclResult_t irecv_v9(void* r, int n, void** d, size_t* sizes, int* tags, void** mh, void** req) {
  return api::irecv(r, n, d, sizes, tags, mh, req);
}
// v10+: NCCL marks LL/LL128 receives, which may complete before their data has landed, by
// presetting *request to NCCL_NET_OPTIONAL_RECV_COMPLETION.
ncclResult_t irecv_v10(void* r, int n, void** d, size_t* sizes, int* tags, void** mh, void**, void** req) {
  const bool optional = req && reinterpret_cast<uintptr_t>(*req) == NCCL_NET_OPTIONAL_RECV_COMPLETION;
  return api::irecv(r, n, d, sizes, tags, mh, req, optional);
}
ncclResult_t iflush(void* r, int n, void** d, int* sizes, void** mh, void** req) { return api::iflush(r, n, d, sizes, mh, req); }
ncclResult_t test(void* req, int* done, int* sizes) { return api::test(req, done, sizes); }
ncclResult_t close_send(void* s) { return api::close_send(s); }
ncclResult_t close_recv(void* r) { return api::close_recv(r); }
ncclResult_t close_listen(void* l) { return api::close_listen(l); }

}  // namespace

// Optional entries (getDeviceMr, irecvConsumed, makeVDevice, setNetAttr) are null: the data path
// runs on the host proxy, there are no device-side net handles and no virtual device merging.
B200NET_EXPORT ncclNet_v6_t ncclNetPlugin_v6 = {
    g_name, init_v6, devices, get_properties_v6, listen_v6, connect_v6, accept_v6, reg_mr_v6, reg_mr_dmabuf, dereg_mr,
    isend_v6, irecv_v6, iflush, test, close_send, close_recv, close_listen};
B200NET_EXPORT ncclNet_v7_t ncclNetPlugin_v7 = {
    g_name, init_v6, devices, get_properties_v7, listen_v6, connect_v7, accept_v7, reg_mr_v6, reg_mr_dmabuf, dereg_mr,
    isend_v6, irecv_v6, iflush, test, close_send, close_recv, close_listen, nullptr, nullptr};
B200NET_EXPORT ncclNet_v8_t ncclNetPlugin_v8 = {
    g_name, init_v6, devices, get_properties_v8, listen_v6, connect_v7, accept_v7, reg_mr_v8, reg_mr_dmabuf, dereg_mr,
    isend_v6, irecv_v6, iflush, test, close_send, close_recv, close_listen, nullptr, nullptr};
B200NET_EXPORT ncclNet_v9_t ncclNetPlugin_v9 = {
    g_name, init_v6, devices, get_properties_v9, listen_v6, connect_v7, accept_v7, reg_mr_v8, reg_mr_dmabuf, dereg_mr,
    isend_v9, irecv_v9, iflush, test, close_send, close_recv, close_listen, nullptr, nullptr, nullptr};
B200NET_EXPORT ncclNet_v10_t ncclNetPlugin_v10 = {
    g_name, init_v10, devices, get_properties_v9, listen_v6, connect_v10, accept_v7, reg_mr_v8, reg_mr_dmabuf, dereg_mr,
    isend_v10, irecv_v10, iflush, test, close_send, close_recv, close_listen, nullptr, nullptr, nullptr};
B200NET_EXPORT ncclNet_v11_t ncclNetPlugin_v11 = {
    g_name, init_v11, devices, get_properties_v11, listen_v11, connect_v11, accept_v7, reg_mr_v8, reg_mr_dmabuf, dereg_mr,
    isend_v10, irecv_v10, iflush, test, close_send, close_recv, close_listen, nullptr, nullptr, nullptr, finalize_v11,
    nullptr};
B200NET_EXPORT ncclNet_v12_t ncclNetPlugin_v12 = {
    g_name, init_v11, devices, get_properties_v12, listen_v11, connect_v11, accept_v7, reg_mr_v8, reg_mr_dmabuf, dereg_mr,
    isend_v10, irecv_v10, iflush, test, close_send, close_recv, close_listen, nullptr, nullptr, nullptr, finalize_v11,
    nullptr};
