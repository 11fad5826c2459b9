#include "b200net/api.h"

#include <sys/stat.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <set>

#include "b200net/histogram.h"
#include "b200net/plugin_stats.h"
#include "b200net/log.h"
#include "b200net/param.h"
#include "b200net/tracepoint.h"

namespace b200net::api {

// Comm objects hold a shared_ptr to their endpoint so it outlives the thread table entry.
static std::mutex g_ep_mu;
static std::map<Comm*, std::shared_ptr<Endpoint>> g_comm_eps;

static void hold(Comm* c, std::shared_ptr<Endpoint> ep) {
  std::lock_guard<std::mutex> g(g_ep_mu);
  g_comm_eps[c] = std::move(ep);
}
static void release(Comm* c) {
  std::lock_guard<std::mutex> g(g_ep_mu);
  g_comm_eps.erase(c);
}

static ncclResult_t check_return(ncclResult_t r) {
  if (r != ncclSuccess && params().abort_on_error.get()) {
    NET_WARN("aborting on error %d (ABORT_ON_ERROR is set)", static_cast<int>(r));
    abort();
  }
  return r;
}

#define API_GUARD_BEGIN try {
#define API_GUARD_END                                                     \
  }                                                                       \
  catch (const std::exception& e) {                                       \
    NET_WARN("caught exception: %s", e.what());                           \
    return check_return(ncclInternalError);                               \
  }                                                                       \
  catch (...) {                                                           \
    NET_WARN("caught unknown exception");                                 \
    return check_return(ncclInternalError);                               \
  }

ncclResult_t init(ncclDebugLogger_t log_fn) {
  API_GUARD_BEGIN
  if (log_fn) set_logger(log_fn);
  trace::enable_from_params();
  Plugin* p = nullptr;
  const int rc = net_create_plugin(&p);
  if (rc != 0) {
    NET_WARN("plugin initialisation failed: %d", rc);
    return check_return(to_nccl(rc));
  }
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t fini() {
  API_GUARD_BEGIN
  net_destroy_plugin();   // endpoints add their byte counts to the totals as they go
  stats::print_all_histograms();
  PluginStats::get().report();
  trace::write_trace_file();
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t devices(int* ndev) {
  if (!ndev) return check_return(ncclInvalidArgument);
  Plugin* p = net_plugin();
  if (!p) return check_return(ncclInvalidUsage);
  *ndev = p->num_devices();
  return ncclSuccess;
}

ncclResult_t get_properties(int dev, Properties* props) {
  API_GUARD_BEGIN
  Plugin* p = net_plugin();
  if (!p) return check_return(ncclInvalidUsage);
  if (!props || dev < 0 || dev >= p->num_devices()) return check_return(ncclInvalidArgument);
  return check_return(to_nccl(p->device(dev)->get_properties(props)));
  API_GUARD_END
}

ncclResult_t listen(int dev, void* handle, void** lcomm) {
  API_GUARD_BEGIN
  Plugin* p = net_plugin();
  if (!p) return check_return(ncclInvalidUsage);
  if (!handle || !lcomm || dev < 0 || dev >= p->num_devices()) return check_return(ncclInvalidArgument);
  *lcomm = nullptr;
  std::shared_ptr<Endpoint> ep = p->device(dev)->get_ep();  // the calling thread's endpoint
  if (!ep || !ep->is_active()) return check_return(ncclSystemError);
  ListenComm* l = nullptr;
  const int rc = ep->listen(static_cast<ConnHandle*>(handle), &l);
  if (rc != 0) return check_return(to_nccl(rc));
  hold(l, ep);
  *lcomm = l;
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t connect(int dev, void* handle, void** scomm, int traffic_class) {
  API_GUARD_BEGIN
  Plugin* p = net_plugin();
  if (!p) return check_return(ncclInvalidUsage);
  if (!handle || !scomm || dev < 0 || dev >= p->num_devices()) return check_return(ncclInvalidArgument);
  *scomm = nullptr;
  auto* h = static_cast<ConnHandle*>(handle);
  // re-entrant: a connect already under way continues on the endpoint that started it
  std::shared_ptr<Endpoint> ep;
  if (h->state.comm) {
    std::lock_guard<std::mutex> g(g_ep_mu);
    auto it = g_comm_eps.find(h->state.comm);
    if (it != g_comm_eps.end()) ep = it->second;
  }
  if (!ep) ep = p->device(dev)->get_ep();
  if (!ep || !ep->is_active()) return check_return(ncclSystemError);
  SendComm* before = h->state.comm;
  SendComm* s = nullptr;
  const int rc = ep->connect(h, &s, traffic_class);
  if (rc != 0) {
    if (before) release(before);
    return check_return(to_nccl(rc));
  }
  if (h->state.comm && h->state.comm != before) hold(h->state.comm, ep);  // connect in progress
  if (s) {
    hold(s, ep);
    *scomm = s;
    PluginStats::bump(PluginStats::get().connects);
  }
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t accept(void* lcomm, void** rcomm) {
  API_GUARD_BEGIN
  if (!lcomm || !rcomm) return check_return(ncclInvalidArgument);
  *rcomm = nullptr;
  auto* l = static_cast<ListenComm*>(lcomm);
  if (!l->ep->is_active()) return check_return(ncclRemoteError);
  RecvComm* r = nullptr;
  const int rc = l->accept(&r);
  if (rc != 0) return check_return(to_nccl(rc));
  if (r) {
    std::shared_ptr<Endpoint> ep;
    {
      std::lock_guard<std::mutex> g(g_ep_mu);
      ep = g_comm_eps[l];
    }
    hold(r, ep);
    *rcomm = r;
    PluginStats::bump(PluginStats::get().accepts);
  }
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t reg_mr(void* comm, void* data, size_t size, int type, void** mhandle) {
  API_GUARD_BEGIN
  if (!comm || !mhandle || (!data && size)) return check_return(ncclInvalidArgument);
  if (type != NCCL_PTR_HOST && type != NCCL_PTR_CUDA) return check_return(ncclInvalidArgument);
  auto* c = static_cast<Comm*>(comm);
  if (!c->ep->is_active()) return check_return(ncclRemoteError);
  MrHandle* mh = nullptr;
  const int rc = c->ep->reg_mr(data, size, type, &mh);
  if (rc != 0) return check_return(to_nccl(rc));
  *mhandle = mh;
  return ncclSuccess;
  API_GUARD_END
}

// A dma-buf descriptor names the allocation that the virtual address already identifies, and peers
// reach the memory through a mapping of that allocation, so the descriptor is not exported. It is
// still held to what it claims: it must be an open descriptor, and when it reports a size (dma-buf
// descriptors answer lseek(SEEK_END)) the registered range must lie inside it.
static int check_dmabuf(int fd, uint64_t offset, size_t size) {
  struct stat st;
  if (fd < 0 || fstat(fd, &st) != 0) return -EBADF;
  const off_t total = lseek(fd, 0, SEEK_END);
  if (total > 0 && (offset > static_cast<uint64_t>(total) || size > static_cast<uint64_t>(total) - offset)) return -EINVAL;
  return 0;
}

ncclResult_t reg_mr_dmabuf(void* comm, void* data, size_t size, int type, uint64_t offset, int fd, void** mhandle) {
  API_GUARD_BEGIN
  if (!comm || !mhandle || (!data && size)) return check_return(ncclInvalidArgument);
  if (type != NCCL_PTR_HOST && type != NCCL_PTR_CUDA) return check_return(ncclInvalidArgument);
  if (const int bad = check_dmabuf(fd, offset, size)) {
    NET_WARN("regMrDmaBuf: descriptor %d does not cover offset %llu + %zu bytes (%d)", fd,
             static_cast<unsigned long long>(offset), size, bad);
    return check_return(ncclInvalidArgument);
  }
  auto* c = static_cast<Comm*>(comm);
  if (!c->ep->is_active()) return check_return(ncclRemoteError);
  MrHandle* mh = nullptr;
  const int rc = c->ep->reg_mr_dmabuf(data, size, type, offset, fd, &mh);
  if (rc != 0) return check_return(to_nccl(rc));
  *mhandle = mh;
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t dereg_mr(void* comm, void* mhandle) {
  API_GUARD_BEGIN
  if (!comm) return check_return(ncclInvalidArgument);
  if (!mhandle) return ncclSuccess;
  auto* c = static_cast<Comm*>(comm);
  return check_return(to_nccl(c->ep->dereg_mr(static_cast<MrHandle*>(mhandle))));
  API_GUARD_END
}

ncclResult_t isend(void* scomm, void* data, size_t size, int tag, void* mhandle, void** request) {
  API_GUARD_BEGIN
  if (!scomm || !request || (!data && size)) return check_return(ncclInvalidArgument);
  *request = nullptr;
  auto* s = static_cast<SendComm*>(scomm);
  Request* r = nullptr;
  const int rc = s->send(data, size, tag, static_cast<MrHandle*>(mhandle), &r);
  if (rc != 0) return check_return(to_nccl(rc));
  PluginStats& st = PluginStats::get();
  if (r) {
    PluginStats::bump(st.sends);
    PluginStats::bump(st.send_bytes, size);
    if (st.histograms_on()) r->t_post_ns = PluginStats::now_ns();
  } else {
    PluginStats::bump(st.send_backoffs);
  }
  *request = r;
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t irecv(void* rcomm, int n, void** data, size_t* sizes, int* tags, void** mhandles, void** request,
                   bool optional_completion) {
  API_GUARD_BEGIN
  if (!rcomm || !request || !data || !sizes || !tags) return check_return(ncclInvalidArgument);
  if (n < 1 || n > NET_MAX_RECVS) {
    NET_WARN("irecv with %d buffers: at most %d receives can be grouped", n, NET_MAX_RECVS);
    return check_return(ncclInvalidArgument);
  }
  *request = nullptr;
  auto* rc_ = static_cast<RecvComm*>(rcomm);
  Request* r = nullptr;
  const int rc = rc_->recv(n, data, sizes, tags, reinterpret_cast<MrHandle**>(mhandles), &r, optional_completion);
  if (rc != 0) return check_return(to_nccl(rc));
  PluginStats::bump(r ? PluginStats::get().recvs : PluginStats::get().recv_backoffs);
  if (r && PluginStats::get().histograms_on()) r->t_post_ns = PluginStats::now_ns();
  *request = r;
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t iflush(void* rcomm, int n, void** data, int* sizes, void** mhandles, void** request) {
  API_GUARD_BEGIN
  if (!rcomm || !request) return check_return(ncclInvalidArgument);
  if (n < 0 || n > NET_MAX_RECVS) return check_return(ncclInvalidArgument);
  *request = nullptr;
  auto* rc_ = static_cast<RecvComm*>(rcomm);
  Request* r = nullptr;
  const int rc = rc_->flush(n, data, sizes, reinterpret_cast<MrHandle**>(mhandles), &r);
  if (rc != 0) return check_return(to_nccl(rc));
  PluginStats::bump(PluginStats::get().flushes);
  *request = r;
  return ncclSuccess;
  API_GUARD_END
}

ncclResult_t test(void* request, int* done, int* sizes) {
  API_GUARD_BEGIN
  if (!request || !done) return check_return(ncclInvalidArgument);
  const int rc = static_cast<Request*>(request)->test(done, sizes);
  if (rc != 0) PluginStats::bump(PluginStats::get().requests_failed);
  return check_return(to_nccl(rc));
  API_GUARD_END
}

ncclResult_t close_send(void* scomm) {
  API_GUARD_BEGIN
  if (!scomm) return check_return(ncclInvalidArgument);
  auto* s = static_cast<SendComm*>(scomm);
  std::shared_ptr<Endpoint> keep;
  {
    std::lock_guard<std::mutex> g(g_ep_mu);
    keep = g_comm_eps[s];
  }
  release(s);
  return check_return(to_nccl(s->close()));
  API_GUARD_END
}
ncclResult_t close_recv(void* rcomm) {
  API_GUARD_BEGIN
  if (!rcomm) return check_return(ncclInvalidArgument);
  auto* r = static_cast<RecvComm*>(rcomm);
  std::shared_ptr<Endpoint> keep;
  {
    std::lock_guard<std::mutex> g(g_ep_mu);
    keep = g_comm_eps[r];
  }
  release(r);
  return check_return(to_nccl(r->close()));
  API_GUARD_END
}
ncclResult_t close_listen(void* lcomm) {
  API_GUARD_BEGIN
  if (!lcomm) return check_return(ncclInvalidArgument);
  auto* l = static_cast<ListenComm*>(lcomm);
  std::shared_ptr<Endpoint> keep;
  {
    std::lock_guard<std::mutex> g(g_ep_mu);
    keep = g_comm_eps[l];
  }
  release(l);
  return check_return(to_nccl(l->close()));
  API_GUARD_END
}

}  // namespace b200net::api
