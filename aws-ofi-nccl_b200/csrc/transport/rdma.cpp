// RDMA-style transport: receiver-driven rendezvous through a control mailbox, multi-rail striped
// writes with completion notifications, an eager path for small messages, grouped receives, a
// retry queue for back-pressured posts, close messages and endpoint abort
// (reference: src/nccl_ofi_rdma.cpp — send() :5646-5877, recv() :3545-3746, test() :2234-2307,
//  the completion loop :1485-1568, pending-request retries :1376-1453, close :3895-4304).
//
// The "wire" is the shared-memory fabric for host buffers and CUDA IPC mappings + copy-engine
// copies on per-rail streams for device buffers; the protocol state machine is independent of it.
#include <sched.h>
#include <unistd.h>

#include <array>
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <deque>
#include <functional>
#include <list>
#include <map>
#include <memory>
#include <set>

#include "b200net/assert.h"
#include "b200net/cm.h"
#include "b200net/cuda_shim.h"
#include "b200net/freelist.h"
#include "b200net/histogram.h"
#include "b200net/ipc_mapper.h"
#include "b200net/log.h"
#include "b200net/msgbuff.h"
#include "b200net/net.h"
#include "b200net/param.h"
#include "b200net/plugin_stats.h"
#include "b200net/net_kernels.h"
#include "b200net/rdma_proto.h"
#include "b200net/scheduler.h"
#include "b200net/shm_fabric.h"
#include "b200net/tracepoint.h"

namespace b200net::rdma {

class RdmaEndpoint;
class RdmaSendComm;
class RdmaRecvComm;

constexpr uint16_t DGRAM_DEVICE_FRAG = static_cast<uint16_t>(DgramType::USER) + 1;
struct DeviceFragHdr {
  uint64_t remote_addr;
  uint32_t len;
  uint32_t pad;
};

// ------------------------------------------------------------------------------------------ requests
struct Stripe {
  int rail;
  size_t offset, len, done;
  cuda::Event event;   // non-null while a copy-engine transfer is in flight
  bool posted, complete, notified;
  int kslot = -1;      // completion slot of a copy-kernel transfer in flight
  std::shared_ptr<std::atomic<int>> job;  // status of a stripe handed to a host copy worker
};

class RdmaSendReq : public Request {
 public:
  int test(int* done, int* sizes) override;
  // A stripe still held by a copy worker reads this request's source buffer: wait for it.
  ~RdmaSendReq() override {
    for (Stripe& s : stripes)
      while (s.job && s.job->load(std::memory_order_acquire) == 0) sched_yield();
  }
  RdmaSendComm* comm = nullptr;
  void* data = nullptr;
  size_t size = 0;
  int tag = 0;
  ReqState state = ReqState::CREATED;
  bool eager = false;       // sent eagerly, waiting to be bound to a control entry
  uint16_t seq = 0;
  uint8_t recv_idx = 0;
  CtrlEntry target{};       // copy of the control entry this send writes into
  std::vector<Stripe> stripes;
  std::vector<uint8_t> bounce;  // host copy of a device source that must travel through host memory
  bool via_frags = false;       // the target registration has an IPC handle that could not be opened here
  uint64_t serial = 0;          // unique per endpoint; queued retries name the request by it
};

struct SubRecv {
  void* buf;
  size_t cap;
  int tag;
  MrHandle* mh;             // only dereferenced while the receive is being posted
  int mem_type = NCCL_PTR_HOST;  // copied then: the registration may be released before an eager payload lands
  size_t received = 0;
  int segs_done = 0, segs_expected = -1;
  bool done = false;
};

class RdmaRecvReq : public Request {
 public:
  int test(int* done, int* sizes) override;
  RdmaRecvComm* comm = nullptr;
  uint16_t seq = 0;
  int n = 0;
  SubRecv subs[MAX_RECVS];
  int ndone = 0;
  bool no_completion = false;   // LL/LL128: NCCL finds the data by polling flags inside the buffer
  bool user_released = false;   // test() already reported done; the object lives until the writes land
  ReqState state = ReqState::PENDING;
};

class RdmaFlushReq : public Request {
 public:
  explicit RdmaFlushReq(RdmaEndpoint* e) : ep(e) {}
  int test(int* done, int* sizes) override;
  RdmaEndpoint* ep;
};

struct EagerRx {  // an eager message that arrived before (or without) a matching posted receive
  EagerHdr hdr;
  std::vector<uint8_t> data;
};

// ------------------------------------------------------------------------------------------ endpoint
class RdmaEndpoint : public Endpoint {
 public:
  RdmaEndpoint(Domain* d, int num_rails);
  ~RdmaEndpoint() override;
  int listen(ConnHandle* handle, ListenComm** lcomm) override;
  int connect(ConnHandle* handle, SendComm** scomm, int traffic_class) override;
  int reg_mr(void* data, size_t size, int type, MrHandle** mh) override;
  int reg_mr_dmabuf(void* data, size_t size, int type, uint64_t offset, int fd, MrHandle** mh) override;
  int dereg_mr(MrHandle* mh) override;

  int progress();
  void handle_dgram(const DgramHdr& h, const void* payload);
  int ensure_published(MrHandle* mh);
  cuda::Stream rail_stream(int rail);
  void* map_peer_cuda(PeerMapping* peer, const MrTableEntry* e);
  // Loads the plugin's device kernels into the current context. Only called from set-up paths
  // (registration, connect, listen): loading a module or a function while a collective kernel
  // that waits for this very transport is running can block forever.
  void prepare_kernels() {
    if (!kernels_tried && cuda::available()) {
      cuda::Context ctx = nullptr;
      if (cuda::ctx_get_current(&ctx) == 0 && ctx) {
        kernels = NetKernels::get();
        kernels_tried = true;
        // streams too are created here, on a set-up path, not by the first send of a collective
        for (int rail = 0; rail < num_rails; ++rail) rail_stream(rail);
      }
    }
  }
  NetKernels* kernels = nullptr;   // null: copy engine only
  bool kernels_tried = false;
  // payload bytes by the path they took (reported when the endpoint goes away)
  uint64_t bytes_kernel = 0, bytes_copy_engine = 0, bytes_staged = 0, bytes_host = 0, bytes_eager = 0;

  FabricEndpoint fab;
  ConnectionManager cm;
  int num_rails;
  IdPool comm_ids{NET_MAX_COMMS};
  std::map<uint32_t, RdmaSendComm*> send_comms;
  std::map<uint32_t, RdmaRecvComm*> recv_comms;
  std::deque<std::function<int()>> pending;  // posts that met a full ring (-EAGAIN); retried in order
  std::vector<cuda::Stream> streams;
  // (peer pid, IPC handle bytes) -> mapped base. Keyed by the handle, not by the MR key: keys are
  // recycled when a buffer is deregistered, and a new registration under an old key is a
  // different allocation.
  std::map<std::pair<uint32_t, std::array<uint8_t, 64>>, std::shared_ptr<IpcMapJob>> ipc_maps;
  bool warned_ipc = false, noted_ipc_wait = false;
  void note_unmapped(PeerMapping* peer, const MrTableEntry* e);
  std::set<std::pair<MrHandle*, int>> published;
  std::map<MrHandle*, int> export_fds;   // descriptors kept open for peers that import a CUDA_VMM registration
  // Requests a queued retry may still touch, by serial number: a request's address can be handed
  // out again (to another communicator's request) while an old retry for it is still queued.
  std::map<uint64_t, RdmaSendReq*> live_send_reqs;
  uint64_t next_req_serial = 1;
  bool in_progress = false;
};

class RdmaListenComm : public ListenComm {
 public:
  int accept(RecvComm** recv) override;
  int close() override;
  std::unique_ptr<CmListener> listener;
  std::unique_ptr<CmReceiver> receiver;  // connection being accepted
  RdmaRecvComm* pending_comm = nullptr;
  CommStage stage = CommStage::COMM_CREATE_START;
};

class RdmaSendComm : public SendComm {
 public:
  ~RdmaSendComm() override;
  int send(void* data, size_t size, int tag, MrHandle* mh, Request** req) override;
  int close() override;
  void bind_eager_queue();
  bool tag_is_queued(int tag) const;
  int start_rendezvous(RdmaSendReq* r, const CtrlEntry& e);
  int post_stripes(RdmaSendReq* r);
  void consume_entry(int idx, int num_recvs);
  RdmaEndpoint* rep() { return static_cast<RdmaEndpoint*>(ep); }

  std::unique_ptr<CmSendConnector> connector;
  std::unique_ptr<ShmWindow> mailbox;  // owned; the receiver maps it and writes control entries
  PeerMapping* peer = nullptr;
  uint16_t next_seq = 0;       // receive group the next send goes to
  uint8_t consumed_mask = 0;   // entries of that group already taken
  uint16_t next_eager_seq = 0;
  std::deque<RdmaSendReq*> eager_queue;
  std::unique_ptr<ThresholdScheduler> sched;
  int inflight = 0;
  uint32_t nonce = 0;
  bool connected = false, peer_closed = false;
};

class RdmaRecvComm : public RecvComm {
 public:
  ~RdmaRecvComm() override;
  int recv(int n, void** data, size_t* sizes, int* tags, MrHandle** mh, Request** req, bool optional) override;
  int flush(int n, void** data, int* sizes, MrHandle** mh, Request** req) override;
  int close() override;
  void on_write_completion(const WriteCompletion& wc);
  void on_eager(const EagerHdr& h, const void* data);
  void match_eager();
  void finish_sub(RdmaRecvReq* r, int idx);
  RdmaEndpoint* rep() { return static_cast<RdmaEndpoint*>(ep); }

  std::unique_ptr<ShmWindow> mailbox;  // sender's mailbox, mapped
  PeerMapping* peer = nullptr;
  uint16_t next_seq = 0;
  std::unique_ptr<MsgBuff> msgbuff;
  std::list<RdmaRecvReq*> posted;      // incomplete receive groups, oldest first
  std::list<EagerRx> eager_rx;         // arrived eager messages in eager_seq order
  uint16_t eager_arrived = 0;          // eager messages with a sequence number before this have all arrived
  uint8_t eager_taken[MAILBOX_SLOTS] = {};  // per group: entries matched to eager messages / completed
  int inflight = 0;
  uint32_t nonce = 0;
  bool peer_closed = false;
};

// ------------------------------------------------------------------------------------------ endpoint impl
RdmaEndpoint::RdmaEndpoint(Domain* d, int rails) : Endpoint(d), cm(&fab), num_rails(rails) {}

RdmaEndpoint::~RdmaEndpoint() {
  {
    PluginStats& st = PluginStats::get();
    PluginStats::bump(st.bytes_kernel, bytes_kernel);
    PluginStats::bump(st.bytes_copy_engine, bytes_copy_engine);
    PluginStats::bump(st.bytes_staged, bytes_staged);
    PluginStats::bump(st.bytes_host, bytes_host);
    PluginStats::bump(st.bytes_eager, bytes_eager);
    for (auto& [k, job] : ipc_maps) {
      const int state = job ? job->state.load(std::memory_order_acquire) : -1;
      PluginStats::bump(state == 1 ? st.ipc_maps : (state == 0 ? st.ipc_map_deferred : st.ipc_map_failures));
    }
  }
  if (bytes_kernel | bytes_copy_engine | bytes_staged | bytes_host | bytes_eager)
    NET_INFO(NCCL_NET, "endpoint payload bytes: copy kernel %llu, copy engine %llu, staged through host %llu, host writes %llu, eager %llu",
             static_cast<unsigned long long>(bytes_kernel), static_cast<unsigned long long>(bytes_copy_engine),
             static_cast<unsigned long long>(bytes_staged), static_cast<unsigned long long>(bytes_host),
             static_cast<unsigned long long>(bytes_eager));
  for (auto& [k, job] : ipc_maps)
    if (job && job->abandon()) job->close_mapping();
  for (auto& [mh, fd] : export_fds) ::close(fd);
  for (auto s : streams)
    if (s) cuda::stream_destroy(s);
}

cuda::Stream RdmaEndpoint::rail_stream(int rail) {
  if (streams.empty()) streams.assign(static_cast<size_t>(num_rails), nullptr);
  rail %= num_rails;
  if (!streams[rail]) {
    if (domain->device->gpu_ordinal >= 0) cuda::ensure_primary_ctx(domain->device->gpu_ordinal);
    if (cuda::stream_create(&streams[rail]) != 0) return nullptr;
  }
  return streams[rail];
}

void* RdmaEndpoint::map_peer_cuda(PeerMapping* peer, const MrTableEntry* e) {
  if (peer->pid == static_cast<uint32_t>(getpid())) return reinterpret_cast<void*>(e->base);  // same process: directly usable
  std::array<uint8_t, 64> handle;
  memcpy(handle.data(), e->ipc_handle, handle.size());
  const auto key = std::make_pair(peer->pid, handle);
  auto it = ipc_maps.find(key);
  if (it == ipc_maps.end()) {
    // first use of this allocation: the open runs on the helper thread (it may wait for the device)
    if (domain->device->gpu_ordinal >= 0) cuda::ensure_primary_ctx(domain->device->gpu_ordinal);
    cuda::Context ctx = nullptr;
    cuda::ctx_get_current(&ctx);
    it = ipc_maps.emplace(key, IpcMapper::instance().submit(e->ipc_handle, ctx, e->kind == static_cast<uint32_t>(MrKind::CUDA_VMM))).first;
    // once an open has outlasted the grace period the device is evidently busy: later first uses
    // stall the caller only briefly (an open that does not have to wait for the device takes microseconds)
    if (it->second) {
      const uint64_t grace = params().ipc_map_wait_us.get();
      IpcMapper::wait(*it->second, noted_ipc_wait ? std::min<uint64_t>(grace, 500) : grace);
    }
  }
  if (!it->second) return nullptr;
  return it->second->state.load(std::memory_order_acquire) == 1 ? it->second->mapped : nullptr;
}
// Says once per endpoint why payloads for a peer's device memory go through host fragments.
void RdmaEndpoint::note_unmapped(PeerMapping* peer, const MrTableEntry* e) {
  std::array<uint8_t, 64> handle;
  memcpy(handle.data(), e->ipc_handle, handle.size());
  auto it = ipc_maps.find(std::make_pair(peer->pid, handle));
  const bool in_progress = it != ipc_maps.end() && it->second && it->second->state.load(std::memory_order_acquire) == 0;
  if (in_progress) {
    if (!noted_ipc_wait) NET_INFO(NCCL_NET, "mapping device memory of process %u is still in progress; payloads are staged through host memory until it arrives", peer->pid);
    noted_ipc_wait = true;
  } else {
    if (!warned_ipc) NET_WARN("device memory of process %u cannot be mapped here; payloads to it are staged through host memory", peer->pid);
    warned_ipc = true;
  }
}
int RdmaEndpoint::ensure_published(MrHandle* mh) {
  if (!mh) return 0;
  if (published.count({mh, 0})) return 0;
  MrTableEntry e;
  memset(&e, 0, sizeof(e));
  e.key = mh->key;
  e.base = reinterpret_cast<uint64_t>(mh->base);
  e.size = mh->size;
  e.kind = static_cast<uint32_t>(mh->kind);
  if (mh->kind == MrKind::CUDA_IPC) {
    void* base = nullptr;
    size_t sz = 0;
    int dev = 0;
    if (cuda::pointer_info(mh->base, &dev, &base, &sz, nullptr) != 0) return -EINVAL;
    e.base = reinterpret_cast<uint64_t>(base);
    e.size = sz;
    e.device = static_cast<uint32_t>(dev);
    if (cuda::ipc_get_handle(base, e.ipc_handle) != 0) {
      mh->kind = MrKind::CUDA_STAGED;
      e.kind = static_cast<uint32_t>(MrKind::CUDA_STAGED);
    }
  } else if (mh->kind == MrKind::CUDA_VMM) {
    // memory of the virtual-memory API (NCCL's own buffers are such): peers import the allocation
    // behind the mapped range through a descriptor that this process keeps open for them
    void* base = nullptr;
    size_t sz = 0;
    int dev = 0, fd = -1;
    const bool ok = cuda::pointer_info(mh->base, &dev, &base, &sz, nullptr) == 0 &&
                    static_cast<char*>(base) + sz >= static_cast<char*>(mh->base) + mh->size &&   // one allocation covers it
                    cuda::vmm_export_range(base, &fd) == 0;
    if (ok) {
      static std::atomic<uint64_t> next_export{1};
      VmmShare sh{VMM_SHARE_MAGIC, fd, static_cast<uint32_t>(getpid()), 0, sz, next_export.fetch_add(1)};
      static_assert(sizeof(sh) <= sizeof(e.ipc_handle), "share record fits the handle bytes");
      memcpy(e.ipc_handle, &sh, sizeof(sh));
      e.base = reinterpret_cast<uint64_t>(base);
      e.size = sz;
      e.device = static_cast<uint32_t>(dev);
      export_fds[mh] = fd;
    } else {
      mh->kind = MrKind::CUDA_STAGED;
      e.kind = static_cast<uint32_t>(MrKind::CUDA_STAGED);
    }
  }
  const int rc = fab.mr_publish(e);
  if (rc == 0) published.insert({mh, 0});
  return rc;
}

int RdmaEndpoint::reg_mr(void* data, size_t size, int type, MrHandle** out) {
  std::lock_guard<std::recursive_mutex> g(ep_lock);
  if (type != NCCL_PTR_HOST) prepare_kernels();
  MrCache* cache = domain->mr_cache.get();
  const MrCacheKey key = MrCacheKey::from_iovec(data, size);
  if (cache) {
    if (void* h = cache->lookup(key)) {
      *out = static_cast<MrHandle*>(h);
      return 0;
    }
  }
  const uint64_t id = domain->mr_keys.allocate();
  if (id == IdPool::ID_NONE) return -ENOSPC;
  auto* mh = new MrHandle();
  mh->key = id + 1;
  mh->base = data;
  mh->size = size;
  mh->type = type;
  mh->domain = domain;
  mh->kind = MrKind::HOST;
  if (type == NCCL_PTR_CUDA) {
    bool vmm = false;
    if (!cuda::available() || cuda::pointer_info(data, nullptr, nullptr, nullptr, &vmm) != 0) {
      domain->mr_keys.free_id(id);
      delete mh;
      return -EINVAL;
    }
    mh->kind = vmm ? MrKind::CUDA_VMM : MrKind::CUDA_IPC;
  }
  if (cache) {
    const int rc = cache->insert(key, mh);
    if (rc != 0 && rc != -EEXIST) {
      domain->mr_keys.free_id(id);
      delete mh;
      return rc;
    }
  }
  B200NET_TRACE_EVENT(GinRegMr, domain->device->dev_id, 0, 0, size, mh);
  *out = mh;
  return 0;
}

int RdmaEndpoint::reg_mr_dmabuf(void* data, size_t size, int type, uint64_t, int, MrHandle** mh) {
  // On NVLink a dma-buf descriptor adds nothing over the virtual address: register the range.
  return reg_mr(data, size, type, mh);
}

int RdmaEndpoint::dereg_mr(MrHandle* mh) {
  std::lock_guard<std::recursive_mutex> g(ep_lock);
  if (!mh) return 0;
  if (MrCache* cache = domain->mr_cache.get()) {
    const int rc = cache->del(mh);
    if (rc == 0) return 0;  // other users remain
  }
  fab.mr_unpublish(mh->key);
  published.erase({mh, 0});
  if (auto fd = export_fds.find(mh); fd != export_fds.end()) {
    ::close(fd->second);
    export_fds.erase(fd);
  }
  domain->mr_keys.free_id(mh->key - 1);
  delete mh;
  return 0;
}

void RdmaEndpoint::handle_dgram(const DgramHdr& h, const void* payload) {
  if (cm.handle_dgram(h, payload)) return;
  switch (h.type) {
    case static_cast<uint16_t>(DgramType::WRITE_COMPLETION): {
      const auto* wc = static_cast<const WriteCompletion*>(payload);
      auto it = recv_comms.find(wc->remote_comm_id);
      if (it != recv_comms.end()) it->second->on_write_completion(*wc);
      break;
    }
    case static_cast<uint16_t>(DgramType::EAGER): {
      const auto* eh = static_cast<const EagerHdr*>(payload);
      auto it = recv_comms.find(eh->remote_comm_id);
      if (it != recv_comms.end()) it->second->on_eager(*eh, static_cast<const char*>(payload) + sizeof(EagerHdr));
      break;
    }
    case static_cast<uint16_t>(DgramType::CLOSE): {
      const auto* cmsg = static_cast<const CloseMsg*>(payload);
      auto r = recv_comms.find(cmsg->remote_comm_id);
      if (r != recv_comms.end() && r->second->nonce == cmsg->nonce) r->second->peer_closed = true;
      auto s = send_comms.find(cmsg->remote_comm_id);
      if (s != send_comms.end() && s->second->nonce == cmsg->nonce) s->second->peer_closed = true;
      break;
    }
    case DGRAM_DEVICE_FRAG: {
      const auto* fh = static_cast<const DeviceFragHdr*>(payload);
      cuda::Stream s = rail_stream(0);
      if (s) {
        cuda::memcpy_async(reinterpret_cast<void*>(fh->remote_addr), static_cast<const char*>(payload) + sizeof(*fh),
                           fh->len, s);
        cuda::stream_synchronize(s);  // the ring cell is recycled on return
      }
      break;
    }
    default:
      NET_INFO(NCCL_NET, "unexpected datagram type %u dropped", h.type);
  }
}

int RdmaEndpoint::progress() {
  if (in_progress) return 0;  // re-entered from a handler
  in_progress = true;
  const int budget = params().cq_read_count.get() * 16;
  B200NET_TRACE_EVENT(ProcessCompletionsRdma, domain->device->dev_id, 0, 0, 0, this);
  fab.poll(budget, [this](const DgramHdr& h, const void* p) { handle_dgram(h, p); });
  // retry queue: strictly in order, stop at the first post that is still back-pressured
  while (!pending.empty()) {
    const int rc = pending.front()();
    if (rc == -EAGAIN) break;
    pending.pop_front();
    B200NET_TRACE_EVENT(PendingQueueRemove, domain->device->dev_id, 0, 0, 0, this);
  }
  in_progress = false;
  return 0;
}

// ------------------------------------------------------------------------------------------ listen / connect / accept
int RdmaEndpoint::listen(ConnHandle* handle, ListenComm** lcomm) {
  std::lock_guard<std::recursive_mutex> g(ep_lock);
  prepare_kernels();
  auto l = std::make_unique<RdmaListenComm>();
  l->ep = this;
  l->dev_id = domain->device->dev_id;
  l->listener = cm.listen();
  if (!l->listener) return -ENOSPC;
  memset(handle, 0, sizeof(*handle));
  strncpy(handle->ep_name, fab.name().c_str(), sizeof(handle->ep_name) - 1);
  handle->comm_id = l->listener->id();
  *lcomm = l.release();
  return 0;
}

int RdmaEndpoint::connect(ConnHandle* handle, SendComm** scomm, int) {
  std::lock_guard<std::recursive_mutex> g(ep_lock);
  prepare_kernels();
  *scomm = nullptr;
  auto* sc = static_cast<RdmaSendComm*>(handle->state.comm);
  if (!sc) {
    const uint64_t id = comm_ids.allocate();
    if (id == IdPool::ID_NONE) return -ENOSPC;
    sc = new RdmaSendComm();
    sc->ep = this;
    sc->dev_id = domain->device->dev_id;
    sc->local_comm_id = static_cast<uint32_t>(id);
    char name[48];
    snprintf(name, sizeof(name), "/b200net.mb.%d.%u.%u", static_cast<int>(getpid()), fab.id(), sc->local_comm_id);
    sc->mailbox = ShmWindow::create(name, MAILBOX_BYTES);
    if (!sc->mailbox) {
      comm_ids.free_id(id);
      delete sc;
      return -ENOMEM;
    }
    sc->sched = std::make_unique<ThresholdScheduler>(num_rails, params().min_stripe_size.get(),
                                                     params().sched_max_small_rr_size.get());
    ConnPayload p;
    memset(&p, 0, sizeof(p));
    p.comm_id = sc->local_comm_id;
    p.num_rails = static_cast<uint32_t>(num_rails);
    sc->nonce = static_cast<uint32_t>(std::chrono::steady_clock::now().time_since_epoch().count()) ^
                (static_cast<uint32_t>(getpid()) << 16) ^ (sc->local_comm_id * 2654435761u);
    p.nonce = sc->nonce;
    strncpy(p.mailbox_name, name, sizeof(p.mailbox_name) - 1);
    const std::string peer_name(handle->ep_name, strnlen(handle->ep_name, sizeof(handle->ep_name)));
    sc->connector = cm.connect(peer_name, handle->comm_id, &p, sizeof(p));
    sc->peer = fab.av_insert(peer_name);
    if (!sc->connector || !sc->peer) {
      comm_ids.free_id(id);
      delete sc;
      return -EHOSTUNREACH;
    }
    send_comms[sc->local_comm_id] = sc;
    handle->state.comm = sc;
    handle->state.stage = CommStage::COMM_SEND_CONN;
  }
  progress();
  const int rc = sc->connector->test_ready();
  if (rc < 0) return rc;
  if (rc == 0) {
    handle->state.stage = CommStage::COMM_CONN_RESP_REQ_PENDING;
    return 0;  // *scomm stays null: call again
  }
  const auto& resp = sc->connector->conn_resp_data();
  if (resp.size() < sizeof(ConnRespPayload)) return -EPROTO;
  sc->remote_comm_id = reinterpret_cast<const ConnRespPayload*>(resp.data())->comm_id;
  sc->connector.reset();
  sc->connected = true;
  handle->state.stage = CommStage::COMM_CONNECTED;
  handle->state.comm = nullptr;
  *scomm = sc;
  return 0;
}

int RdmaListenComm::accept(RecvComm** out) {
  auto* e = static_cast<RdmaEndpoint*>(ep);
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *out = nullptr;
  e->progress();
  if (stage == CommStage::COMM_CREATE_START || stage == CommStage::COMM_CONN_REQ_PENDING) {
    receiver = listener->accept();
    if (!receiver) {
      stage = CommStage::COMM_CONN_REQ_PENDING;
      return 0;
    }
    const auto& msg = receiver->conn_msg_data();
    if (msg.size() < sizeof(ConnPayload)) return -EPROTO;
    const auto* p = reinterpret_cast<const ConnPayload*>(msg.data());
    const uint64_t id = e->comm_ids.allocate();
    if (id == IdPool::ID_NONE) return -ENOSPC;
    auto* rc = new RdmaRecvComm();
    rc->ep = e;
    rc->dev_id = dev_id;
    rc->local_comm_id = static_cast<uint32_t>(id);
    rc->remote_comm_id = p->comm_id;
    rc->nonce = p->nonce;
    rc->mailbox = ShmWindow::open(std::string(p->mailbox_name, strnlen(p->mailbox_name, sizeof(p->mailbox_name))));
    rc->peer = e->fab.av_insert(receiver->peer_ep_name());
    if (!rc->mailbox || rc->mailbox->size() < MAILBOX_BYTES || !rc->peer) {
      e->comm_ids.free_id(id);
      delete rc;
      return -EHOSTUNREACH;
    }
    rc->msgbuff = std::make_unique<MsgBuff>(MAILBOX_SLOTS, SEQ_BITS, 0);
    e->recv_comms[rc->local_comm_id] = rc;
    ConnRespPayload resp{rc->local_comm_id, static_cast<uint32_t>(e->num_rails)};
    receiver->set_conn_resp_msg_data(&resp, sizeof(resp));
    pending_comm = rc;
    stage = CommStage::COMM_CONN_RESP_REQ_PENDING;
  }
  if (stage == CommStage::COMM_CONN_RESP_REQ_PENDING) {
    const int rc = receiver->test_ready();
    if (rc < 0) return rc;
    if (rc == 0) return 0;
    *out = pending_comm;
    pending_comm = nullptr;
    receiver.reset();
    stage = CommStage::COMM_CREATE_START;  // ready for the next connection on this listener
  }
  return 0;
}

int RdmaListenComm::close() {
  auto* e = static_cast<RdmaEndpoint*>(ep);
  {
    std::lock_guard<std::recursive_mutex> g(e->ep_lock);
    if (pending_comm) {
      e->recv_comms.erase(pending_comm->local_comm_id);
      e->comm_ids.free_id(pending_comm->local_comm_id);
      delete pending_comm;
    }
    receiver.reset();
    listener.reset();
  }
  delete this;
  return 0;
}

// ------------------------------------------------------------------------------------------ send side
RdmaSendComm::~RdmaSendComm() = default;

void RdmaSendComm::consume_entry(int idx, int num_recvs) {
  consumed_mask |= static_cast<uint8_t>(1u << idx);
  if (__builtin_popcount(consumed_mask) >= num_recvs) {
    next_seq = (next_seq + 1) & SEQ_MASK;
    consumed_mask = 0;
  }
}


// Bind queued eager sends to control entries that have arrived. The queue is walked in send order
// against the current receive group: a send whose tag has no free entry in that group stays
// queued for a later group while sends behind it (necessarily of other tags) may still fill this
// one; when the group is complete the walk starts over on the next. Sends of one tag therefore
// never overtake each other, and every send lands in the first group, at or after the one that was
// current when it left, that has a free entry of its tag: the rule the receiver applies too.
void RdmaSendComm::bind_eager_queue() {
  auto* box = static_cast<CtrlMsg*>(mailbox->data());
  auto it = eager_queue.begin();
  while (it != eager_queue.end()) {
    RdmaSendReq* r = *it;
    int n = 0;
    const int idx = match_entry(box[next_seq % MAILBOX_SLOTS], next_seq, consumed_mask, r->tag, &n);
    if (idx == -1) return;   // the group has not arrived yet
    if (idx < 0) {           // no free entry of this tag here
      ++it;
      continue;
    }
    r->seq = next_seq;
    r->recv_idx = static_cast<uint8_t>(idx);
    r->state = ReqState::COMPLETED;
    B200NET_TRACE_EVENT(SendEagerComplete, dev_id, local_comm_id, r->seq, r->size, r);
    const uint16_t before = next_seq;
    it = eager_queue.erase(it);
    consume_entry(idx, n);
    if (next_seq != before) it = eager_queue.begin();
  }
}

bool RdmaSendComm::tag_is_queued(int tag) const {
  for (const RdmaSendReq* r : eager_queue)
    if (r->tag == tag) return true;
  return false;
}

int RdmaSendComm::post_stripes(RdmaSendReq* r) {
  RdmaEndpoint* e = rep();
  const MrTableEntry* mr = FabricEndpoint::mr_lookup(peer, r->target.mr_key);
  const uint32_t kind = r->via_frags ? static_cast<uint32_t>(MrKind::CUDA_STAGED)
                                     : (mr ? mr->kind : static_cast<uint32_t>(MrKind::HOST));
  const bool src_dev = !r->bounce.empty() ? false : !cuda::is_host_pointer(r->data);
  const char* src = r->bounce.empty() ? static_cast<const char*>(r->data) : reinterpret_cast<const char*>(r->bounce.data());
  bool all_done = true;
  bool back_pressure = false;   // some ring was full: the post must be retried in order
  for (Stripe& s : r->stripes) {
    if (!s.complete) {
      if (kind == static_cast<uint32_t>(MrKind::CUDA_IPC) || kind == static_cast<uint32_t>(MrKind::CUDA_VMM)) {
        if (!s.posted) {
          void* mapped = e->map_peer_cuda(peer, mr);
          cuda::Stream st = e->rail_stream(s.rail);
          if (!mapped || !st) return -EIO;
          char* dst = static_cast<char*>(mapped) + (r->target.buff_addr - mr->base) + s.offset;
          // device source: the plugin's own copy kernel moves the stripe over NVLink and sets a
          // completion word in pinned memory; anything else goes through the copy engine
          NetKernels* nk = src_dev ? e->kernels : nullptr;
          if (nk && nk->copy_flag(dst, src + s.offset, s.len, st, 0, &s.kslot) == 0) {
            e->bytes_kernel += s.len;
          } else {
            e->bytes_copy_engine += s.len;
            s.kslot = -1;
            if (cuda::event_create(&s.event) != 0 || cuda::memcpy_async(dst, src + s.offset, s.len, st) != 0 ||
                cuda::event_record(s.event, st) != 0)
              return -EIO;
          }
          s.posted = true;
          B200NET_TRACE_EVENT(SendWriteSegmentStart, dev_id, local_comm_id, r->seq, s.len, r);
        }
        if (s.kslot >= 0) {
          NetKernels* nk = e->kernels;
          if (!nk) return -EIO;
          if (nk->done(s.kslot)) {
            nk->release(s.kslot);
            s.kslot = -1;
            s.done = s.len;
            s.complete = true;
          }
        } else {
          const int q = cuda::event_query(s.event);
          if (q < 0) return -EIO;
          if (q == 0) {
            cuda::event_destroy(s.event);
            s.event = nullptr;
            s.done = s.len;
            s.complete = true;
          }
        }
      } else if (kind == static_cast<uint32_t>(MrKind::CUDA_STAGED)) {
        // the target cannot be mapped here: ship fragments that the receiver copies to the device
        const size_t chunk = FAB_LARGE_CELL - sizeof(DeviceFragHdr) - 64;
        while (s.done < s.len) {
          const size_t nbytes = std::min(chunk, s.len - s.done);
          DeviceFragHdr fh{r->target.buff_addr + s.offset + s.done, static_cast<uint32_t>(nbytes), 0};
          // the large ring even for a short tail: the completion is ordered behind it there
          const int rc = e->fab.send(peer, static_cast<DgramType>(DGRAM_DEVICE_FRAG), DGRAM_FLAG_ORDER_AFTER_FRAGS, &fh, sizeof(fh),
                                     src + s.offset + s.done, nbytes);
          if (rc == -EAGAIN) {
            back_pressure = true;
            break;
          }
          if (rc != 0) return rc;
          s.done += nbytes;
          e->bytes_staged += nbytes;
        }
        s.complete = s.done >= s.len;
      } else {
        if (!s.posted) {
          s.posted = true;
          B200NET_TRACE_EVENT(SendWriteSegmentStart, dev_id, local_comm_id, r->seq, s.len, r);
        }
        if (s.job) {
          // a copy worker has this stripe
          const int st = s.job->load(std::memory_order_acquire);
          if (st < 0) return st == -ESRCH ? -ENOTCONN : -EFAULT;
          if (st == 1) {
            s.done = s.len;
            s.complete = true;
            s.job.reset();
          }
        } else if (s.done == 0 && s.len >= params().host_copy_min_size.get() && peer->pid != static_cast<uint32_t>(getpid()) &&
                   !e->fab.writes_are_staged(peer) && [&] {
                     auto status = std::make_shared<std::atomic<int>>(0);
                     if (!HostCopyPool::instance().submit(peer->pid, r->target.buff_addr + s.offset, src + s.offset, s.len, status))
                       return false;
                     s.job = std::move(status);
                     return true;
                   }()) {
          e->bytes_host += s.len;
        } else {
          const size_t before = s.done;
          const int rc = e->fab.write_host(peer, r->target.buff_addr + s.offset, src + s.offset, s.len, &s.done);
          e->bytes_host += s.done - before;
          if (rc != 0 && rc != -EAGAIN) return rc;
          if (rc == -EAGAIN) back_pressure = true;
          s.complete = (rc == 0);
        }
      }
    }
    if (s.complete && !s.notified) {
      WriteCompletion wc{remote_comm_id, r->seq, r->recv_idx, static_cast<uint8_t>(r->stripes.size()), s.len};
      // data that travelled as fragments must be applied before its completion is seen
      const bool staged = kind == static_cast<uint32_t>(MrKind::CUDA_STAGED) ||
                          (kind == static_cast<uint32_t>(MrKind::HOST) && e->fab.writes_are_staged(peer));
      const int rc = e->fab.send(peer, DgramType::WRITE_COMPLETION, staged ? DGRAM_FLAG_ORDER_AFTER_FRAGS : 0, &wc,
                                 sizeof(wc));
      if (rc == 0) {
        s.notified = true;
        B200NET_TRACE_EVENT(SendWriteSegmentComplete, dev_id, local_comm_id, r->seq, s.len, r);
      } else if (rc != -EAGAIN) {
        return rc;
      } else {
        back_pressure = true;
      }
    }
    if (!s.notified) all_done = false;
  }
  if (all_done) {
    r->state = ReqState::COMPLETED;
    return 0;
  }
  // -EAGAIN: a ring was full, retry in order. -EINPROGRESS: only the request's own copies (kernel,
  // copy engine, copy worker) are outstanding; test() polls them, nothing has to be queued.
  return back_pressure ? -EAGAIN : -EINPROGRESS;
}

int RdmaSendComm::start_rendezvous(RdmaSendReq* r, const CtrlEntry& e) {
  r->target.buff_addr = e.buff_addr;
  r->target.mr_key = e.mr_key;
  r->target.buff_len = e.buff_len;
  r->target.flags = e.flags;
  if (r->size > e.buff_len) r->size = e.buff_len;  // a send larger than the posted receive is truncated
  const MrTableEntry* mr = FabricEndpoint::mr_lookup(peer, e.mr_key);
  const bool dst_host = !mr || mr->kind == static_cast<uint32_t>(MrKind::HOST);
  const bool mappable = mr && (mr->kind == static_cast<uint32_t>(MrKind::CUDA_IPC) || mr->kind == static_cast<uint32_t>(MrKind::CUDA_VMM));
  if (mappable && !rep()->map_peer_cuda(peer, mr)) {
    // the peer's device memory cannot be mapped into this process (another container, a driver
    // without IPC): the payload travels as fragments that the receiver copies to its device
    rep()->note_unmapped(peer, mr);
    r->via_frags = true;
  }
  if ((dst_host || r->via_frags || (mr && mr->kind == static_cast<uint32_t>(MrKind::CUDA_STAGED))) && r->size &&
      !cuda::is_host_pointer(r->data)) {
    // device source, destination only reachable through host memory: bounce once
    r->bounce.resize(r->size);
    cuda::Stream st = rep()->rail_stream(0);
    if (!st || cuda::memcpy_async(r->bounce.data(), r->data, r->size, st) != 0 || cuda::stream_synchronize(st) != 0)
      return -EIO;
  }
  Schedule* sc = sched->get_schedule(r->size, rep()->num_rails);
  if (!sc) return -ENOMEM;
  for (size_t i = 0; i < sc->num_xfer_infos; ++i)
    r->stripes.push_back(Stripe{sc->xfers[i].rail_id, sc->xfers[i].offset, sc->xfers[i].msg_size, 0, nullptr, false,
                                false, false});
  sched->release_schedule(sc);
  r->state = ReqState::PENDING;
  return 0;
}

int RdmaSendComm::send(void* data, size_t size, int tag, MrHandle*, Request** req) {
  RdmaEndpoint* e = rep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *req = nullptr;
  if (!e->is_active()) return -ECONNABORTED;
  if (peer_closed) return -ENOTCONN;
  e->progress();
  if (inflight >= NET_MAX_SEND_REQUESTS) return 0;
  bind_eager_queue();
  auto* box = static_cast<CtrlMsg*>(mailbox->data());
  int n = 0;
  // a send may take an entry directly unless an eager send of the same tag is still waiting for
  // one (it has to go first); then it queues behind that one (-3: eager if small, else refused)
  const int idx = tag_is_queued(tag) ? -3 : match_entry(box[next_seq % MAILBOX_SLOTS], next_seq, consumed_mask, tag, &n);
  NET_TRACE(NCCL_NET, "send: seq %u idx %d eagerq %zu ready0 %x size %zu", next_seq, idx, eager_queue.size(),
            box[next_seq % MAILBOX_SLOTS].entries[0].ready.load(), size);
  if (idx >= 0) {
    auto* r = new RdmaSendReq();
    r->comm = this;
    r->data = data;
    r->size = size;
    r->tag = tag;
    r->seq = next_seq;
    r->recv_idx = static_cast<uint8_t>(idx);
    const int rc = start_rendezvous(r, box[next_seq % MAILBOX_SLOTS].entries[idx]);
    if (rc != 0) {
      delete r;
      return rc;
    }
    B200NET_TRACE_EVENT(Send, dev_id, local_comm_id, r->seq, r->size, r);
    PluginStats::bump(PluginStats::get().rendezvous_sends);
    consume_entry(idx, n);
    bind_eager_queue();   // if that completed the group, queued sends may fit the next one
    ++inflight;
    r->serial = e->next_req_serial++;
    e->live_send_reqs[r->serial] = r;
    const int prc = post_stripes(r);
    if (prc != 0 && prc != -EAGAIN && prc != -EINPROGRESS) {
      r->state = ReqState::ERROR;
    } else if (prc == -EAGAIN) {
      B200NET_TRACE_EVENT(PendingQueueInsert, dev_id, local_comm_id, r->seq, r->size, r);
      e->pending.push_back([this, e, r, serial = r->serial]() {
        auto live = e->live_send_reqs.find(serial);
        if (live == e->live_send_reqs.end() || live->second != r || r->state != ReqState::PENDING) return 0;
        const int rc2 = post_stripes(r);
        if (rc2 != 0 && rc2 != -EAGAIN && rc2 != -EINPROGRESS) r->state = ReqState::ERROR;
        return rc2 == -EAGAIN ? -EAGAIN : 0;
      });
    }
    *req = r;
    return 0;
  }
  // no control message yet: eager if allowed
  const size_t eager_max = params().eager_max_size.get();
  const bool eager_size_ok = eager_max > 0 && size <= eager_max && size + sizeof(EagerHdr) <= FAB_LARGE_CELL &&
                             static_cast<int>(eager_queue.size()) < MAX_EAGER_PENDING;
  const void* eager_src = data;
  int eager_slot = -1;
  NetKernels* nk = nullptr;
  std::vector<uint8_t> eager_bounce;
  if (eager_size_ok && size > 0 && !cuda::is_host_pointer(data)) {
    // device payload: the pack kernel writes header + payload + flag into a pinned slot and the
    // datagram is sent from there; without the kernels the copy engine fetches the payload
    nk = size <= NetKernels::EAGER_PAYLOAD_MAX ? e->kernels : nullptr;
    cuda::Stream st = e->rail_stream(0);
    if (!st) return -EIO;
    if (nk && nk->eager_pack(data, size, next_eager_seq, size, st, &eager_slot) == 0) {
      const auto t0 = std::chrono::steady_clock::now();
      while (!nk->eager_done(eager_slot)) {
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(2)) {
          // the slot stays reserved: the kernel may still write it
          NET_WARN("eager pack kernel did not complete within 2 s");
          return -EIO;
        }
      }
      eager_src = nk->eager_slot(eager_slot) + 16;
    } else {
      eager_slot = -1;
      eager_bounce.resize(size);
      if (cuda::memcpy_async(eager_bounce.data(), data, size, st) != 0 || cuda::stream_synchronize(st) != 0) return -EIO;
      eager_src = eager_bounce.data();
    }
  }
  if (eager_size_ok) {
    EagerHdr h;
    memset(&h, 0, sizeof(h));
    h.remote_comm_id = remote_comm_id;
    h.eager_seq = next_eager_seq;
    h.base_seq = next_seq;
    h.base_mask = consumed_mask;
    h.tag = tag;
    h.size = size;
    const int rc = e->fab.send(peer, DgramType::EAGER, 0, &h, sizeof(h), eager_src, size);
    if (eager_slot >= 0) nk->eager_release(eager_slot);  // the datagram holds a copy
    if (rc == 0) {
      e->bytes_eager += size;
      PluginStats::bump(PluginStats::get().eager_sends);
    }
    if (rc == -EAGAIN) return 0;  // ring full: NCCL calls again
    if (rc != 0) return rc;
    auto* r = new RdmaSendReq();
    r->comm = this;
    r->data = data;
    r->size = size;
    r->tag = tag;
    r->eager = true;
    r->state = ReqState::PENDING;
    ++next_eager_seq;
    ++inflight;
    eager_queue.push_back(r);
    B200NET_TRACE_EVENT(SendEagerStart, dev_id, local_comm_id, h.eager_seq, size, r);
    *req = r;
    return 0;
  }
  return 0;  // neither control message nor eager: *req stays null and NCCL retries
}

int RdmaSendReq::test(int* done, int* sizes) {
  RdmaEndpoint* e = comm->rep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *done = 0;
  if (!e->is_active()) return -ECONNABORTED;
  e->progress();
  if (state == ReqState::PENDING && eager) comm->bind_eager_queue();
  if (state == ReqState::PENDING && !eager) {
    const int rc = comm->post_stripes(this);
    if (rc != 0 && rc != -EAGAIN && rc != -EINPROGRESS) state = ReqState::ERROR;
  }
  if (state == ReqState::ERROR) {
    --comm->inflight;
    e->live_send_reqs.erase(serial);
    delete this;
    return -EIO;
  }
  if (state == ReqState::COMPLETED) {
    *done = 1;
    if (sizes) sizes[0] = static_cast<int>(size);
    B200NET_TRACE_EVENT(SendEnd, comm->dev_id, comm->local_comm_id, seq, size, this);
    if (PluginStats::get().histograms_on()) PluginStats::get().sample_send(size, stripes.size(), PluginStats::since(t_post_ns));
    --comm->inflight;
    e->live_send_reqs.erase(serial);
    delete this;
  }
  return 0;
}

int RdmaSendComm::close() {
  RdmaEndpoint* e = rep();
  {
    std::lock_guard<std::recursive_mutex> g(e->ep_lock);
    if (inflight > 0) {
      // requests still in flight: the endpoint's queues reference them, so it cannot be reused
      NET_WARN("send communicator %u closed with %d requests in flight: endpoint aborted", local_comm_id, inflight);
      e->invalidate();
      e->pending.clear();
    }
    if (!params().disable_close_message.get() && peer && connected) {
      CloseMsg m{remote_comm_id, nonce};
      e->fab.send(peer, DgramType::CLOSE, 0, &m, sizeof(m));
    }
    e->send_comms.erase(local_comm_id);
    e->comm_ids.free_id(local_comm_id);
  }
  delete this;
  return 0;
}

// ------------------------------------------------------------------------------------------ receive side
RdmaRecvComm::~RdmaRecvComm() = default;

void RdmaRecvComm::finish_sub(RdmaRecvReq* r, int idx) {
  if (r->subs[idx].done) return;
  r->subs[idx].done = true;
  eager_taken[r->seq % MAILBOX_SLOTS] |= static_cast<uint8_t>(1u << idx);
  if (++r->ndone == r->n) {
    r->state = ReqState::COMPLETED;
    MsgStatus st;
    msgbuff->complete(r->seq, &st);
    posted.remove(r);
    if (r->user_released) delete r;
  }
}

void RdmaRecvComm::on_write_completion(const WriteCompletion& wc) {
  void* elem = nullptr;
  MsgElemType ty;
  MsgStatus st;
  if (msgbuff->retrieve(wc.seq, &elem, &ty, &st) != MsgResult::SUCCESS || ty != MsgElemType::REQ) {
    NET_WARN("write completion for sequence %u with no receive posted (status %d)", wc.seq, static_cast<int>(st));
    return;
  }
  auto* r = static_cast<RdmaRecvReq*>(elem);
  if (wc.recv_idx >= r->n) return;
  SubRecv& s = r->subs[wc.recv_idx];
  s.received += wc.len;
  s.segs_expected = wc.seg_cnt;
  B200NET_TRACE_EVENT(RecvSegmentComplete, dev_id, local_comm_id, wc.seq, wc.len, r);
  if (++s.segs_done >= s.segs_expected) finish_sub(r, wc.recv_idx);
}

void RdmaRecvComm::on_eager(const EagerHdr& h, const void* data) {
  EagerRx rx;
  rx.hdr = h;
  rx.data.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + h.size);
  // keep the list ordered by eager_seq (datagrams of one sender arrive in order; be safe anyway)
  auto it = eager_rx.end();
  while (it != eager_rx.begin()) {
    auto prev = std::prev(it);
    if (static_cast<int16_t>(h.eager_seq - prev->hdr.eager_seq) >= 0) break;
    it = prev;
  }
  eager_rx.insert(it, std::move(rx));
  // eager_arrived: every message sent before it is here (they arrive in order; a gap would hold
  // later ones back until it is filled)
  for (bool advanced = true; advanced;) {
    advanced = false;
    for (const EagerRx& m : eager_rx)
      if (m.hdr.eager_seq == eager_arrived) {
        ++eager_arrived;
        advanced = true;
      }
  }
  B200NET_TRACE_EVENT(EagerRecv, dev_id, local_comm_id, h.eager_seq, h.size, nullptr);
  match_eager();
}

// Repeat the sender's binding rule. Eager messages are taken in the order they were sent; each goes
// to the first posted group, at or after the group that was current when it left (base_seq), that
// has a free entry of its tag: free means taken neither by a send before it (base_mask, for the
// base group) nor by an eager message matched here. A message that finds no such entry yet waits,
// and so does every later message of the same tag; messages of other tags go on.
void RdmaRecvComm::match_eager() {
  int blocked_tags[MAX_EAGER_PENDING + 1];
  int nblocked = 0;
  auto it = eager_rx.begin();
  while (it != eager_rx.end()) {
    EagerRx& rx = *it;
    if (static_cast<int16_t>(rx.hdr.eager_seq - eager_arrived) >= 0) return;  // an earlier one is still missing
    bool blocked = false;
    for (int k = 0; k < nblocked; ++k) blocked = blocked || blocked_tags[k] == rx.hdr.tag;
    RdmaRecvReq* target = nullptr;
    int target_idx = -1;
    if (!blocked) {
      for (RdmaRecvReq* r : posted) {
        if (seq_before(r->seq, rx.hdr.base_seq)) continue;  // the sender had moved past this group
        uint8_t taken = eager_taken[r->seq % MAILBOX_SLOTS];
        if (r->seq == rx.hdr.base_seq) taken |= rx.hdr.base_mask;
        for (int i = 0; i < r->n && !target; ++i) {
          if (!(taken & (1u << i)) && r->subs[i].tag == rx.hdr.tag) {
            target = r;
            target_idx = i;
          }
        }
        if (target) break;
      }
    }
    if (!target) {
      if (!blocked && nblocked < MAX_EAGER_PENDING + 1) blocked_tags[nblocked++] = rx.hdr.tag;
      ++it;
      continue;
    }
    SubRecv& s = target->subs[target_idx];
    const size_t nbytes = std::min<size_t>(rx.hdr.size, s.cap);
    if (nbytes) {
      if (s.mem_type == NCCL_PTR_CUDA) {
        cuda::Stream st = rep()->rail_stream(0);
        if (st) {
          cuda::memcpy_async(s.buf, rx.data.data(), nbytes, st);
          cuda::stream_synchronize(st);
        }
      } else {
        memcpy(s.buf, rx.data.data(), nbytes);
      }
    }
    s.received = nbytes;
    it = eager_rx.erase(it);
    finish_sub(target, target_idx);
  }
}

int RdmaRecvComm::recv(int n, void** data, size_t* sizes, int* tags, MrHandle** mh, Request** req, bool optional) {
  RdmaEndpoint* e = rep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *req = nullptr;
  if (!e->is_active()) return -ECONNABORTED;
  if (n < 1 || n > MAX_RECVS) return -EINVAL;
  e->progress();
  if (inflight >= NET_MAX_REQUESTS) return 0;
  // the mailbox slot of this sequence number must not still describe a live group
  const uint16_t seq = next_seq;
  auto* r = new RdmaRecvReq();
  r->comm = this;
  r->seq = seq;
  r->n = n;
  r->no_completion = optional && params().early_completion.get();
  MsgStatus st;
  if (msgbuff->insert(seq, r, MsgElemType::REQ, &st) != MsgResult::SUCCESS) {
    delete r;
    return 0;  // window full: try again after completions
  }
  eager_taken[seq % MAILBOX_SLOTS] = 0;
  auto* box = static_cast<CtrlMsg*>(mailbox->data());
  CtrlMsg& slot = box[seq % MAILBOX_SLOTS];
  B200NET_TRACE_EVENT(WriteCtrlStart, dev_id, local_comm_id, seq, n, r);
  for (int i = 0; i < n; ++i) {
    r->subs[i] = SubRecv{data[i], sizes[i], tags[i], mh ? mh[i] : nullptr, (mh && mh[i]) ? mh[i]->type : NCCL_PTR_HOST};
    if (mh && mh[i]) {
      const int rc = e->ensure_published(mh[i]);
      if (rc != 0) {
        msgbuff->complete(seq, &st);
        delete r;
        return rc;
      }
    }
    CtrlEntry& c = slot.entries[i];
    c.buff_addr = reinterpret_cast<uint64_t>(data[i]);
    c.mr_key = (mh && mh[i]) ? mh[i]->key : 0;
    c.buff_len = sizes[i];
    c.tag = tags[i];
    c.flags = r->no_completion ? CTRL_FLAG_NO_COMPLETION : 0;
    c.num_recvs = static_cast<uint8_t>(n);
    c.recv_idx = static_cast<uint8_t>(i);
  }
  // publish back to front so that entry 0 becoming ready implies the others are written
  for (int i = n - 1; i >= 0; --i)
    slot.entries[i].ready.store(static_cast<uint16_t>(CTRL_READY | (seq & SEQ_MASK)), std::memory_order_release);
  B200NET_TRACE_EVENT(WriteCtrlEnd, dev_id, local_comm_id, seq, n, r);
  B200NET_TRACE_EVENT(Recv, dev_id, local_comm_id, seq, n, r);
  next_seq = (next_seq + 1) & SEQ_MASK;
  ++inflight;
  posted.push_back(r);
  match_eager();
  *req = r;
  return 0;
}

int RdmaRecvReq::test(int* done, int* sizes) {
  RdmaEndpoint* e = comm->rep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *done = 0;
  if (!e->is_active()) return -ECONNABORTED;
  e->progress();
  if (state == ReqState::COMPLETED) {
    *done = 1;
    if (sizes)
      for (int i = 0; i < n; ++i) sizes[i] = static_cast<int>(subs[i].received);
    B200NET_TRACE_EVENT(RecvEnd, comm->dev_id, comm->local_comm_id, seq, n, this);
    {
      size_t total = 0;
      for (int i = 0; i < n; ++i) total += subs[i].received;
      PluginStats::bump(PluginStats::get().recv_bytes, total);
      if (PluginStats::get().histograms_on()) PluginStats::get().sample_recv(total, PluginStats::since(t_post_ns));
    }
    --comm->inflight;
    delete this;
  } else if (no_completion) {
    // early completion: report the posted sizes now, retire the bookkeeping when the writes land
    *done = 1;
    if (sizes)
      for (int i = 0; i < n; ++i) sizes[i] = static_cast<int>(subs[i].cap);
    --comm->inflight;
    user_released = true;
  }
  return 0;
}

int RdmaFlushReq::test(int* done, int*) {
  std::lock_guard<std::recursive_mutex> g(ep->ep_lock);
  ep->progress();
  *done = 1;
  delete this;
  return 0;
}

// Data written by a peer becomes visible to this GPU once the completion has been observed with
// acquire semantics (NVLink has no ordering hole like PCIe posted writes): a fence is enough. The
// driver flush is used when CUDA_FLUSH_ENABLE asks for it and the driver offers it.
int RdmaRecvComm::flush(int n, void**, int* sizes, MrHandle** mh, Request** req) {
  RdmaEndpoint* e = rep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *req = nullptr;
  if (!e->is_active()) return -ECONNABORTED;
  bool any = false;
  for (int i = 0; i < n; ++i)
    if (sizes && sizes[i] > 0 && mh && mh[i] && mh[i]->type == NCCL_PTR_CUDA) any = true;
  B200NET_TRACE_EVENT(Flush, dev_id, local_comm_id, 0, static_cast<uint64_t>(n), this);
  std::atomic_thread_fence(std::memory_order_acq_rel);
  if (any && params().cuda_flush_enable.get()) cuda::flush_gpudirect_rdma_writes();
  *req = new RdmaFlushReq(e);
  return 0;
}

int RdmaRecvComm::close() {
  RdmaEndpoint* e = rep();
  {
    std::lock_guard<std::recursive_mutex> g(e->ep_lock);
    if (inflight > 0) {
      NET_WARN("receive communicator %u closed with %d requests in flight: endpoint aborted", local_comm_id, inflight);
      e->invalidate();
      e->pending.clear();
    }
    if (!params().disable_close_message.get() && peer) {
      CloseMsg m{remote_comm_id, nonce};
      e->fab.send(peer, DgramType::CLOSE, 0, &m, sizeof(m));
    }
    // invalidate the control entries so that a sender never acts on a dead group
    auto* box = static_cast<CtrlMsg*>(mailbox->data());
    for (int s = 0; s < MAILBOX_SLOTS; ++s)
      for (int i = 0; i < MAX_RECVS; ++i) box[s].entries[i].ready.store(0, std::memory_order_release);
    e->recv_comms.erase(local_comm_id);
    e->comm_ids.free_id(local_comm_id);
  }
  delete this;
  return 0;
}

// ------------------------------------------------------------------------------------------ domain / device
class RdmaDomain : public Domain {
 public:
  RdmaDomain(Device* d, int rails) : Domain(d), rails_(rails) {}
  std::shared_ptr<Endpoint> create_endpoint() override { return std::make_shared<RdmaEndpoint>(this, rails_); }

 private:
  int rails_;
};

class RdmaDevice : public Device {
 public:
  RdmaDevice(int id, std::string n, int rails, int gpu) : Device(id, std::move(n)), rails_(rails) { gpu_ordinal = gpu; }
  std::shared_ptr<Domain> create_domain() override { return std::make_shared<RdmaDomain>(this, rails_); }
  int get_properties(Properties* p) override;

 private:
  int rails_;
};

int RdmaDevice::get_properties(Properties* p) {
  const int rc = fill_common_properties(this, p, rails_);
  if (rc) return rc;
  p->max_recvs = NET_MAX_RECVS;
  p->reg_is_global = 1;
  // one message may be any size: stripes are bounded by the scheduler, not by a transfer limit
  p->max_p2p_bytes = static_cast<size_t>(INT32_MAX);
  p->max_coll_bytes = static_cast<size_t>(INT32_MAX);
  p->num_rails = rails_;
  return 0;
}

}  // namespace b200net::rdma

namespace b200net {
int rdma_create_devices(Plugin* p, int ndev, int num_rails) {
  const int ngpu = cuda::device_count();
  for (int i = 0; i < ndev; ++i) {
    char name[64];
    snprintf(name, sizeof(name), "nvl%d", i);
    p->devices.push_back(std::make_unique<rdma::RdmaDevice>(i, name, num_rails, i < ngpu ? i : -1));
  }
  p->protocol = "RDMA";
  return 0;
}
}  // namespace b200net
