// Exported GIN and RMA tables: ncclGinPlugin_v11 / v13 (host proxy), ncclGinPlugin_v14
// (kernel-initiated: set-up only), ncclRmaPlugin_v14 / v15 (host-initiated put / get / signal)
// (reference: src/rdma/gin/nccl_ofi_gin_api.cpp:566-754, nccl_ofi_gin_gdaki.cpp:1175-1243).
#include <cstring>
#include <mutex>
#include <set>

#include "b200net/api.h"
#include "b200net/gin.h"
#include "b200net/gin_dev_handle.h"
#include "b200net/log.h"
#include "b200net/platform.h"

using namespace b200net;
using namespace b200net::gin;
#define B200NET_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

std::mutex g_mu;
int g_refs = 0;
std::set<CollComm*> g_comms;

ncclResult_t gin_init(void** ctx, uint64_t, ncclDebugLogger_t log_fn) {
  std::lock_guard<std::mutex> g(g_mu);
  // GIN rides on the net transport's domain: bring the net plugin up (reference counted)
  const ncclResult_t r = api::init(log_fn);
  if (r != ncclSuccess) return r;
  ++g_refs;
  if (ctx) *ctx = &g_refs;
  return ncclSuccess;
}
ncclResult_t gin_finalize(void*) {
  std::lock_guard<std::mutex> g(g_mu);
  if (g_refs <= 0) return ncclInvalidUsage;
  --g_refs;
  return api::fini();
}
ncclResult_t gin_devices(int* n) { return api::devices(n); }

template <typename P>
ncclResult_t fill_props(int dev, P* out, ncclNetDeviceType type) {
  if (!out) return ncclInvalidArgument;
  Properties p;
  const ncclResult_t r = api::get_properties(dev, &p);
  if (r != ncclSuccess) return r;
  static std::mutex mu;
  static std::string names[64], pcis[64];
  std::lock_guard<std::mutex> g(mu);
  names[dev % 64] = p.name;
  pcis[dev % 64] = p.pci_path;
  memset(out, 0, sizeof(*out));
  out->name = const_cast<char*>(names[dev % 64].c_str());
  out->pciPath = pcis[dev % 64].empty() ? nullptr : const_cast<char*>(pcis[dev % 64].c_str());
  out->guid = p.guid;
  out->ptrSupport = p.ptr_support;
  out->regIsGlobal = p.reg_is_global;
  out->forceFlush = 0;
  out->speed = p.port_speed_mbps;
  out->port = p.port;
  out->latency = p.latency_us;
  out->maxComms = GIN_MAX_COMMS;
  out->maxRecvs = 1;
  out->netDeviceType = type;
  out->netDeviceVersion = 1;
  out->vProps.ndevs = 1;
  out->vProps.devs[0] = dev;
  out->maxP2pBytes = p.max_p2p_bytes;
  out->maxCollBytes = p.max_coll_bytes;
  out->maxMultiRequestSize = 1;
  return ncclSuccess;
}
ncclResult_t props_v11(int dev, ncclNetProperties_v11_t* out) { return fill_props(dev, out, NCCL_NET_DEVICE_GIN_PROXY); }
ncclResult_t props_v12_proxy(int dev, ncclNetProperties_v12_t* out) {
  const ncclResult_t r = fill_props(dev, out, NCCL_NET_DEVICE_GIN_PROXY);
  if (r == ncclSuccess) out->railId = out->planeId = -1;
  return r;
}
ncclResult_t props_v12_kernel(int dev, ncclNetProperties_v12_t* out) {
  const ncclResult_t r = fill_props(dev, out, NCCL_NET_DEVICE_GIN_GDAKI);
  if (r == ncclSuccess) out->railId = out->planeId = -1;
  return r;
}

ncclResult_t gin_listen(void*, int dev, void* handle, void** lcomm) {
  if (!handle || !lcomm) return ncclInvalidArgument;
  auto* l = new gin::ListenComm();
  l->dev = dev;
  const ncclResult_t r = api::listen(dev, handle, &l->net_listen);
  if (r != ncclSuccess) {
    delete l;
    return r;
  }
  *lcomm = l;
  return ncclSuccess;
}

ncclResult_t gin_connect(void*, void* handles[], int nranks, int rank, void* lcomm, void** coll) {
  if (!handles || !lcomm || !coll || nranks < 1 || rank < 0 || rank >= nranks) return ncclInvalidArgument;
  auto* l = static_cast<gin::ListenComm*>(lcomm);
  try {
    auto* c = new CollComm(l->dev, nranks, rank);
    const int rc = c->connect(handles, l);
    if (rc != 0) {
      delete c;
      return api::to_nccl(rc);
    }
    {
      std::lock_guard<std::mutex> g(g_mu);
      g_comms.insert(c);
    }
    *coll = c;
    return ncclSuccess;
  } catch (const std::exception& e) {
    NET_WARN("GIN connect failed: %s", e.what());
    return ncclSystemError;
  }
}
ncclResult_t gin_connect_v11(void* ctx, void* handles[], int nranks, int rank, void* lcomm, void** coll) {
  return gin_connect(ctx, handles, nranks, rank, lcomm, coll);
}

ncclResult_t gin_close_listen(void* lcomm) {
  if (!lcomm) return ncclInvalidArgument;
  auto* l = static_cast<gin::ListenComm*>(lcomm);
  const ncclResult_t r = api::close_listen(l->net_listen);
  delete l;
  return r;
}
ncclResult_t gin_close_coll(void* coll) {
  if (!coll) return ncclInvalidArgument;
  auto* c = static_cast<CollComm*>(coll);
  const int rc = c->close();
  {
    std::lock_guard<std::mutex> g(g_mu);
    g_comms.erase(c);
  }
  delete c;
  return api::to_nccl(rc);
}

// ---- registration ---------------------------------------------------------------------------------
ncclResult_t reg_mr_sym(void* coll, void* data, size_t size, int type, uint64_t flags, void** mh, void** gin_handle) {
  if (!coll || !mh || (!data && size)) return ncclInvalidArgument;
  if (type != NCCL_PTR_HOST && type != NCCL_PTR_CUDA) return ncclInvalidArgument;
  SymmMr* m = nullptr;
  const int rc = static_cast<CollComm*>(coll)->reg_mr_sym(data, size, type, flags, &m);
  if (rc != 0) return api::to_nccl(rc);
  *mh = m;
  if (gin_handle) *gin_handle = m;
  return ncclSuccess;
}
ncclResult_t reg_mr_sym_dmabuf(void* coll, void* data, size_t size, int type, uint64_t, int, uint64_t flags, void** mh,
                               void** gin_handle) {
  return reg_mr_sym(coll, data, size, type, flags, mh, gin_handle);
}
// Kernel-initiated mode: the gin handle is the device address of a GinDevWindow (where every rank's
// registered range is mapped on this GPU, and its size), which the device API takes next to the
// context's GinDevHandle (reference: the regMrSym block, src/rdma/gin/nccl_ofi_gin_gdaki.cpp:950-1164).
ncclResult_t reg_mr_sym_kernel(void* coll, void* data, size_t size, int type, uint64_t flags, void** mh, void** gin_handle) {
  const ncclResult_t r = reg_mr_sym(coll, data, size, type, flags, mh, nullptr);
  if (r != ncclSuccess) return r;
  auto* m = static_cast<SymmMr*>(*mh);
  auto* c = static_cast<CollComm*>(coll);
  if (!m->gpu_handle_block && type == NCCL_PTR_CUDA) {
    if (c->nranks > b200::GIN_MAX_RANKS) return ncclInvalidArgument;
    b200::GinDevWindow w;
    memset(&w, 0, sizeof(w));
    for (int i = 0; i < c->nranks; ++i) w.base[i] = static_cast<uint8_t*>(m->mapped[i]);
    w.bytes = size;
    if (cuda::mem_alloc(&m->gpu_handle_block, sizeof(w)) != 0) return ncclSystemError;
    cuda::Stream st = nullptr;
    cuda::stream_create(&st);
    cuda::memcpy_async(m->gpu_handle_block, &w, sizeof(w), st);
    cuda::stream_synchronize(st);
    cuda::stream_destroy(st);
  }
  if (gin_handle) *gin_handle = m->gpu_handle_block;
  return ncclSuccess;
}
ncclResult_t reg_mr_sym_dmabuf_kernel(void* coll, void* data, size_t size, int type, uint64_t, int, uint64_t flags,
                                      void** mh, void** gin_handle) {
  return reg_mr_sym_kernel(coll, data, size, type, flags, mh, gin_handle);
}
ncclResult_t dereg_mr_sym(void* coll, void* mh) {
  if (!coll) return ncclInvalidArgument;
  return api::to_nccl(static_cast<CollComm*>(coll)->dereg_mr_sym(static_cast<SymmMr*>(mh)));
}
ncclResult_t rma_reg_mr_sym(void* coll, void* data, size_t size, int type, uint64_t flags, void** mh) {
  return reg_mr_sym(coll, data, size, type, flags, mh, nullptr);
}
ncclResult_t rma_reg_mr_sym_dmabuf(void* coll, void* data, size_t size, int type, uint64_t, int, uint64_t flags, void** mh) {
  return reg_mr_sym(coll, data, size, type, flags, mh, nullptr);
}

// ---- contexts ------------------------------------------------------------------------------------
ncclResult_t create_context_common(void* coll, int n_sig, int n_cnt, int n_ctx, bool kernel, void** gin_ctx,
                                   ncclNetDeviceHandle_t** dev_handle) {
  if (!coll || !gin_ctx) return ncclInvalidArgument;
  GinContext* c = nullptr;
  const int rc = static_cast<CollComm*>(coll)->create_context(n_sig, n_cnt, n_ctx, kernel, &c);
  if (rc != 0) return api::to_nccl(rc);
  *gin_ctx = c;
  if (dev_handle) *dev_handle = &c->net_dev_handle;
  return ncclSuccess;
}
ncclResult_t create_context_v11(void* coll, int n_sig, int n_cnt, void** gin_ctx, ncclNetDeviceHandle_t** dh) {
  return create_context_common(coll, n_sig, n_cnt, 1, false, gin_ctx, dh);
}
ncclResult_t create_context_v13(void* coll, ncclGinConfig_v13_t* cfg, void** gin_ctx, ncclNetDeviceHandle_t** dh) {
  if (!cfg) return ncclInvalidArgument;
  if (cfg->nContexts > GIN_MAX_CONTEXTS) return ncclInvalidArgument;
  return create_context_common(coll, cfg->nSignals, cfg->nCounters, cfg->nContexts, false, gin_ctx, dh);
}
// The configuration is validated before the communicator pointer is touched at all, so a caller
// probing the supported backend versions may pass any pointer there.
ncclResult_t create_context_v14(void* coll, ncclGinConfig_v14_t* cfg, void** gin_ctx, ncclNetDeviceHandle_t** dh) {
  if (!cfg) return ncclInvalidArgument;
  if (cfg->backendVersion < 0 || cfg->backendVersion > GIN_MAX_BACKEND_VERSION) {
    NET_WARN("GIN backend version %d not supported (0..%d)", cfg->backendVersion, GIN_MAX_BACKEND_VERSION);
    return ncclInvalidArgument;
  }
  if (cfg->nContexts < 1 || cfg->nContexts > GIN_MAX_CONTEXTS) return ncclInvalidArgument;
  Platform* plat = PlatformManager::instance().get_platform();
  if (!plat || !plat->gdaki_capable()) return ncclInvalidUsage;
  return create_context_common(coll, cfg->nSignals, cfg->nCounters, cfg->nContexts, true, gin_ctx, dh);
}
ncclResult_t destroy_context(void* gin_ctx) {
  if (!gin_ctx) return ncclInvalidArgument;
  auto* c = static_cast<GinContext*>(gin_ctx);
  return api::to_nccl(c->comm->destroy_context(c));
}
ncclResult_t rma_create_context(void* coll, ncclRmaConfig_t* cfg, void** rma_ctx) {
  if (!cfg) return ncclInvalidArgument;
  return create_context_common(coll, 0, 0, cfg->nContexts < 1 ? 1 : cfg->nContexts, false, rma_ctx, nullptr);
}

// ---- operations (v11 takes the communicator, v13+ the context) ---------------------------------------
ncclResult_t put_common(CollComm* c, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh, uint32_t rank,
                        bool with_sig, uint64_t sig_off, void* sig_mh, uint64_t sig_val, uint32_t sig_op, void** req) {
  if (!c || !req) return ncclInvalidArgument;
  GinRequest* r = nullptr;
  const int rc = c->iput(so, static_cast<SymmMr*>(smh), size, d_off, static_cast<SymmMr*>(dmh), rank, with_sig, sig_off,
                         static_cast<SymmMr*>(sig_mh), sig_val, sig_op, &r);
  if (rc != 0) return api::to_nccl(rc);
  *req = r;
  return ncclSuccess;
}
ncclResult_t iput_v11(void* coll, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh, uint32_t rank, void** req) {
  return put_common(static_cast<CollComm*>(coll), so, smh, size, d_off, dmh, rank, false, 0, nullptr, 0, 0, req);
}
ncclResult_t iput_signal_v11(void* coll, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh, uint32_t rank,
                             uint64_t sig_off, void* sig_mh, uint64_t sig_val, uint32_t sig_op, void** req) {
  return put_common(static_cast<CollComm*>(coll), so, smh, size, d_off, dmh, rank, true, sig_off, sig_mh, sig_val, sig_op, req);
}
CollComm* comm_of(void* ctx) { return ctx ? static_cast<GinContext*>(ctx)->comm : nullptr; }
ncclResult_t iput_v13(void* ctx, int, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh, uint32_t rank, void** req) {
  return put_common(comm_of(ctx), so, smh, size, d_off, dmh, rank, false, 0, nullptr, 0, 0, req);
}
ncclResult_t iput_signal_v13(void* ctx, int, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh, uint32_t rank,
                             uint64_t sig_off, void* sig_mh, uint64_t sig_val, uint32_t sig_op, void** req) {
  return put_common(comm_of(ctx), so, smh, size, d_off, dmh, rank, true, sig_off, sig_mh, sig_val, sig_op, req);
}
ncclResult_t iget_v13(void* ctx, int, uint64_t ro, void* rmh, size_t size, uint64_t lo, void* lmh, uint32_t rank, void** req) {
  CollComm* c = comm_of(ctx);
  if (!c || !req) return ncclInvalidArgument;
  GinRequest* r = nullptr;
  const int rc = c->iget(ro, static_cast<SymmMr*>(rmh), size, lo, static_cast<SymmMr*>(lmh), rank, &r);
  if (rc != 0) return api::to_nccl(rc);
  *req = r;
  return ncclSuccess;
}
ncclResult_t iflush_v13(void* ctx, int, void*, uint32_t, void** req) {
  CollComm* c = comm_of(ctx);
  if (!c || !req) return ncclInvalidArgument;
  GinRequest* r = nullptr;
  const int rc = c->iflush(&r);
  if (rc != 0) return api::to_nccl(rc);
  *req = r;
  return ncclSuccess;
}
// RMA adds a strong-signal flag and (v15) option flags; signals here are always applied after the
// data they follow, so "strong" needs nothing extra, and request aggregation is accepted as a hint.
ncclResult_t rma_iput_v14(void* ctx, int c, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh, uint32_t rank, void** req) {
  return iput_v13(ctx, c, so, smh, size, d_off, dmh, rank, req);
}
ncclResult_t rma_iput_signal_v14(void* ctx, int c, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh,
                                 uint32_t rank, uint64_t sig_off, void* sig_mh, uint64_t sig_val, uint32_t sig_op, bool,
                                 void** req) {
  return iput_signal_v13(ctx, c, so, smh, size, d_off, dmh, rank, sig_off, sig_mh, sig_val, sig_op, req);
}
ncclResult_t rma_iput_v15(void* ctx, int c, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh, uint32_t rank,
                          uint32_t, void** req) {
  return iput_v13(ctx, c, so, smh, size, d_off, dmh, rank, req);
}
ncclResult_t rma_iput_signal_v15(void* ctx, int c, uint64_t so, void* smh, size_t size, uint64_t d_off, void* dmh,
                                 uint32_t rank, uint64_t sig_off, void* sig_mh, uint64_t sig_val, uint32_t sig_op, bool,
                                 uint32_t, void** req) {
  return iput_signal_v13(ctx, c, so, smh, size, d_off, dmh, rank, sig_off, sig_mh, sig_val, sig_op, req);
}
ncclResult_t rma_iget_v15(void* ctx, int c, uint64_t ro, void* rmh, size_t size, uint64_t lo, void* lmh, uint32_t rank,
                          uint32_t, void** req) {
  return iget_v13(ctx, c, ro, rmh, size, lo, lmh, rank, req);
}

ncclResult_t gin_test(void*, void* request, int* done) {
  if (!request || !done) return ncclInvalidArgument;
  return api::to_nccl(static_cast<GinRequest*>(request)->test(done));
}
ncclResult_t progress_comm(void* coll) {
  if (!coll) return ncclInvalidArgument;
  return api::to_nccl(static_cast<CollComm*>(coll)->progress());
}
ncclResult_t progress_ctx(void* ctx) { return progress_comm(comm_of(ctx)); }
ncclResult_t query_last_error(void* ctx, bool* has_error) {
  if (!ctx || !has_error) return ncclInvalidArgument;
  auto* c = static_cast<GinContext*>(ctx);
  *has_error = c->has_error || c->comm->has_error();
  return ncclSuccess;
}
// Kernel-initiated mode has no host-side completion path on which an error could surface.
ncclResult_t query_last_error_kernel(void* ctx, bool* has_error) {
  if (!ctx || !has_error) return ncclInvalidArgument;
  *has_error = false;
  return ncclSuccess;
}
ncclResult_t gin_properties_v14(ncclGinProperties_v14_t* p) {
  if (!p) return ncclInvalidArgument;
  p->supportsStrongSignals = false;
  p->supportsVASignals = false;
  return ncclSuccess;
}

}  // namespace

B200NET_EXPORT ncclGin_v11_t ncclGinPlugin_v11 = {
    "B200NVL", gin_init, gin_devices, props_v11, gin_listen, gin_connect_v11, create_context_v11, reg_mr_sym,
    reg_mr_sym_dmabuf, dereg_mr_sym, destroy_context, gin_close_coll, gin_close_listen, iput_v11, iput_signal_v11, gin_test,
    progress_comm, query_last_error, gin_finalize};
B200NET_EXPORT ncclGin_v13_t ncclGinPlugin_v13 = {
    "B200NVL", gin_init, gin_devices, props_v12_proxy, gin_listen, gin_connect, create_context_v13, reg_mr_sym,
    reg_mr_sym_dmabuf, dereg_mr_sym, destroy_context, gin_close_coll, gin_close_listen, iput_v13, iput_signal_v13, iget_v13,
    iflush_v13, gin_test, progress_ctx, query_last_error, gin_finalize};
B200NET_EXPORT ncclGin_v14_t ncclGinPlugin_v14 = {
    "B200NVL_GDAKI", gin_init, gin_devices, gin_properties_v14, props_v12_kernel, gin_listen, gin_connect, create_context_v14,
    reg_mr_sym_kernel, reg_mr_sym_dmabuf_kernel, dereg_mr_sym, destroy_context, gin_close_coll, gin_close_listen,
    progress_ctx, query_last_error_kernel, gin_finalize};
B200NET_EXPORT ncclRma_v14_t ncclRmaPlugin_v14 = {
    "B200NVL", gin_init, gin_devices, props_v12_proxy, gin_listen, gin_connect, rma_create_context, rma_reg_mr_sym,
    rma_reg_mr_sym_dmabuf, dereg_mr_sym, destroy_context, gin_close_coll, gin_close_listen, rma_iput_v14,
    rma_iput_signal_v14, iget_v13, iflush_v13, gin_test, progress_ctx, query_last_error, gin_finalize};
B200NET_EXPORT ncclRma_v15_t ncclRmaPlugin_v15 = {
    "B200NVL", gin_init, gin_devices, props_v12_proxy, gin_listen, gin_connect, rma_create_context, rma_reg_mr_sym,
    rma_reg_mr_sym_dmabuf, dereg_mr_sym, destroy_context, gin_close_coll, gin_close_listen, rma_iput_v15,
    rma_iput_signal_v15, rma_iget_v15, iflush_v13, gin_test, progress_ctx, query_last_error, gin_finalize};
