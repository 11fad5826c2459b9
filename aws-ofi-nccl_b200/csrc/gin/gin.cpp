#include "b200net/gin.h"
#include "b200net/gin_dev_handle.h"
#include "b200net/ipc_mapper.h"

#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstring>

#include "b200net/api.h"
#include "b200net/log.h"
#include "b200net/net_kernels.h"
#include "b200net/param.h"
#include "b200net/plugin_stats.h"
#include "b200net/tracepoint.h"

namespace b200net::gin {

using Clock = std::chrono::steady_clock;
static bool expired(Clock::time_point t0, int seconds = 30) { return Clock::now() - t0 > std::chrono::seconds(seconds); }
static std::atomic<uint32_t> g_next_comm_id{1};

// ------------------------------------------------------------------------------------------ device signal worker
DeviceSignalWorker& DeviceSignalWorker::instance() {
  static DeviceSignalWorker* w = new DeviceSignalWorker();
  return *w;
}
DeviceSignalWorker::DeviceSignalWorker() { thread_ = std::thread([this] { run(); }); }
DeviceSignalWorker::~DeviceSignalWorker() {
  stop_.store(true);
  if (thread_.joinable()) thread_.join();
}
bool DeviceSignalWorker::submit(const SignalWork& w) {
  if (!ctx_.load(std::memory_order_acquire)) {
    cuda::Context cur = nullptr;
    if (cuda::ctx_get_current(&cur) == 0 && cur) ctx_.store(cur, std::memory_order_release);
  }
  if (!ring_.push(w)) return false;
  submitted_.fetch_add(1);
  return true;
}
void DeviceSignalWorker::drain() {
  const uint64_t target = submitted_.load();
  while (completed_.load() < target) std::this_thread::yield();
}
void DeviceSignalWorker::run() {
  int idle = 0;
  while (!stop_.load(std::memory_order_relaxed)) {
    // take a batch, fold additions to the same word, apply each word once
    std::map<uint64_t, uint64_t> batch;
    int n = 0;
    SignalWork w;
    while (n < 512 && ring_.pop(w)) {
      batch[w.addr] += w.value;
      ++n;
    }
    if (!n) {
      if (++idle > 1000) std::this_thread::sleep_for(std::chrono::microseconds(50));
      continue;
    }
    idle = 0;
    if (!stream_) {
      if (void* ctx = ctx_.load(std::memory_order_acquire)) cuda::ctx_set_current(ctx);
      else cuda::ensure_primary_ctx(0);
      cuda::stream_create(&stream_);
    }
    // With the plugin's kernels loaded a signal is an atomic add on the device: it composes with
    // signals that kernels raise on the same word. The host shadow below is the path of a run
    // without the kernels; it owns the word (an update made by anybody else would be lost).
    NetKernels* nk = NetKernels::get();
    if (nk) {
      bool all = true;
      for (auto& [addr, add] : batch) all = all && nk->signal_add(reinterpret_cast<void*>(addr), add, stream_) == 0;
      if (all) {
        cuda::stream_synchronize(stream_);
        completed_.fetch_add(static_cast<uint64_t>(n));
        continue;
      }
      cuda::stream_synchronize(stream_);   // some launch failed: fall through to the copy path for the whole batch is not
                                           // possible (part was applied), so report nothing lost and stop using kernels
      NET_WARN("signal kernel launch failed; %d signal update(s) of this batch may be missing", n);
      completed_.fetch_add(static_cast<uint64_t>(n));
      continue;
    }
    for (auto& [addr, add] : batch) {
      auto it = shadow_.find(addr);
      if (it == shadow_.end()) {
        uint64_t cur = 0;  // first touch: read the word once; afterwards the shadow is authoritative
        cuda::memcpy_async(&cur, reinterpret_cast<void*>(addr), 8, stream_);
        cuda::stream_synchronize(stream_);
        it = shadow_.emplace(addr, cur).first;
      }
      it->second += add;
      cuda::memcpy_async(reinterpret_cast<void*>(addr), &it->second, 8, stream_);
    }
    cuda::stream_synchronize(stream_);
    completed_.fetch_add(static_cast<uint64_t>(n));
  }
}

// ------------------------------------------------------------------------------------------ requests
class StatusRequest : public GinRequest {
 public:
  StatusRequest(CollComm* c, std::shared_ptr<std::atomic<int>> s) : comm(c), status(std::move(s)) {}
  int test(int* done) override {
    comm->progress();
    const int v = status->load();
    *done = v != 0;
    if (v < 0) {
      delete this;
      return v;
    }
    if (v) delete this;
    return 0;
  }
  CollComm* comm;
  std::shared_ptr<std::atomic<int>> status;
};

// ------------------------------------------------------------------------------------------ CollComm
CollComm::CollComm(int dev_, int nranks_, int rank_) : dev(dev_), nranks(nranks_), rank(rank_) {
  comm_id = g_next_comm_id.fetch_add(1);
  peers_.resize(static_cast<size_t>(nranks));
}

CollComm::~CollComm() {
  for (SymmMr* m : mrs_) delete m;
  for (GinContext* c : contexts_) delete c;
}

// A fragment of a put whose target is device memory that the sender cannot map (no IPC handle for
// it, or the mapping failed): the owner copies it to its device when it polls.
constexpr uint16_t GIN_DEVICE_FRAG = static_cast<uint16_t>(DgramType::USER) + 2;
struct GinDeviceFragHdr {
  uint32_t comm_id;
  uint32_t len;
  uint64_t addr;
};

// Blocking helpers over the net transport's own API (used only during collective set-up).
template <typename Idle>
static int net_send_recv(void* scomm, void* rcomm, const void* sbuf, void* rbuf, size_t n, Idle&& idle) {
  void *smh = nullptr, *rmh = nullptr;
  if (api::reg_mr(scomm, const_cast<void*>(sbuf), n, NCCL_PTR_HOST, &smh) != ncclSuccess) return -EIO;
  if (api::reg_mr(rcomm, rbuf, n, NCCL_PTR_HOST, &rmh) != ncclSuccess) return -EIO;
  void *sreq = nullptr, *rreq = nullptr;
  size_t sz = n;
  int tag = 0x61;
  const auto t0 = Clock::now();
  int sdone = 0, rdone = 0;
  while (!sdone || !rdone) {
    if (!rreq && api::irecv(rcomm, 1, &rbuf, &sz, &tag, &rmh, &rreq) != ncclSuccess) return -EIO;
    if (!sreq && api::isend(scomm, const_cast<void*>(sbuf), n, tag, smh, &sreq) != ncclSuccess) return -EIO;
    if (sreq && !sdone && api::test(sreq, &sdone, nullptr) != ncclSuccess) return -EIO;
    if (rreq && !rdone && api::test(rreq, &rdone, nullptr) != ncclSuccess) return -EIO;
    if (expired(t0)) return -ETIMEDOUT;
    idle();
  }
  api::dereg_mr(scomm, smh);
  api::dereg_mr(rcomm, rmh);
  return 0;
}

int CollComm::all_gather(void* buf, size_t bytes) {
  if (nranks == 1) return 0;
  char* b = static_cast<char*>(buf);
  // step s: pass on the block received in step s-1 (own block first); n-1 steps
  for (int s = 0; s < nranks - 1; ++s) {
    const int send_idx = (rank - s + nranks) % nranks;
    const int recv_idx = (rank - s - 1 + nranks) % nranks;
    // While this rank waits inside a collective call, peers may still have operations in flight
    // that need it (a read it has to serve, signals to apply, acknowledgements): keep the engine
    // turning, as a caller without a progress thread of its own cannot.
    const int rc = net_send_recv(ring_send_, ring_recv_, b + send_idx * bytes, b + recv_idx * bytes, bytes, [this] {
      if (!peers_.empty() && peers_[0].map) progress();
    });
    if (rc) return rc;
  }
  return 0;
}

int CollComm::connect(void* handles[], ListenComm* lcomm) {
  std::lock_guard<std::recursive_mutex> g(lock);
  if (nranks > 1) {
    const int next = (rank + 1) % nranks;
    const auto t0 = Clock::now();
    char handle_copy[NCCL_NET_HANDLE_MAXSIZE];
    memcpy(handle_copy, handles[next], sizeof(handle_copy));
    while (!ring_send_ || !ring_recv_) {
      if (!ring_send_ && api::connect(dev, handle_copy, &ring_send_, -1) != ncclSuccess) return -EHOSTUNREACH;
      if (!ring_recv_ && api::accept(lcomm->net_listen, &ring_recv_) != ncclSuccess) return -EHOSTUNREACH;
      if (expired(t0)) return -ETIMEDOUT;
    }
  }
  std::vector<PeerRecord> recs(static_cast<size_t>(nranks));
  memset(recs.data(), 0, recs.size() * sizeof(PeerRecord));
  strncpy(recs[rank].ep_name, fab_.name().c_str(), FAB_EP_NAME_LEN - 1);
  recs[rank].pid = static_cast<uint32_t>(getpid());
  recs[rank].comm_id = comm_id;
  const int rc = all_gather(recs.data(), sizeof(PeerRecord));
  if (rc) return rc;
  for (int r = 0; r < nranks; ++r) {
    peers_[r].map = fab_.av_insert(std::string(recs[r].ep_name, strnlen(recs[r].ep_name, FAB_EP_NAME_LEN)));
    peers_[r].comm_id = recs[r].comm_id;
    if (!peers_[r].map) return -EHOSTUNREACH;
  }
  B200NET_TRACE_EVENT(GinConnect, dev, comm_id, 0, static_cast<uint64_t>(nranks), this);
  return 0;
}

int CollComm::reg_mr_sym(void* data, size_t size, int type, uint64_t flags, SymmMr** out) {
  std::lock_guard<std::recursive_mutex> g(lock);
  for (SymmMr* m : mrs_) {  // the same buffer registered again: share the registration
    if (m->base == data && m->size == size) {
      ++m->refcnt;
      *out = m;
      return 0;
    }
  }
  auto* m = new SymmMr();
  m->base = data;
  m->size = size;
  m->type = type;
  m->flags = flags;
  m->remote.resize(static_cast<size_t>(nranks));
  RemoteMr mine;
  memset(&mine, 0, sizeof(mine));
  mine.addr = reinterpret_cast<uint64_t>(data);
  mine.size = size;
  mine.kind = static_cast<uint32_t>(MrKind::HOST);
  if (type == NCCL_PTR_CUDA) {
    void* base = nullptr;
    size_t sz = 0;
    int d = 0;
    bool vmm = false;
    if (!cuda::available() || cuda::pointer_info(data, &d, &base, &sz, &vmm) != 0) {
      delete m;
      return -EINVAL;
    }
    mine.device = static_cast<uint32_t>(d);
    mine.kind = static_cast<uint32_t>(MrKind::CUDA_STAGED);
    if (!vmm && cuda::ipc_get_handle(base, mine.ipc_handle) == 0) {
      mine.kind = static_cast<uint32_t>(MrKind::CUDA_IPC);
      mine.key = reinterpret_cast<uint64_t>(base);  // allocation base: offsets are taken from it
    } else if (vmm && static_cast<char*>(base) + sz >= static_cast<char*>(data) + size &&
               cuda::vmm_export_range(base, &m->export_fd) == 0) {
      // memory of the virtual-memory API backed by one allocation: peers import it through a descriptor
      static std::atomic<uint64_t> next_export{1};
      VmmShare sh{VMM_SHARE_MAGIC, m->export_fd, static_cast<uint32_t>(getpid()), 0, sz, next_export.fetch_add(1)};
      memcpy(mine.ipc_handle, &sh, sizeof(sh));
      mine.kind = static_cast<uint32_t>(MrKind::CUDA_VMM);
      mine.key = reinterpret_cast<uint64_t>(base);
    }
  }
  m->remote[rank] = mine;
  const int rc = all_gather(m->remote.data(), sizeof(RemoteMr));
  if (rc) {
    if (m->export_fd >= 0) ::close(m->export_fd);
    delete m;
    return rc;
  }
  m->mapped.assign(static_cast<size_t>(nranks), nullptr);
  m->mapped_bytes.assign(static_cast<size_t>(nranks), 0);
  if (type == NCCL_PTR_CUDA) {
    for (int r = 0; r < nranks; ++r) {
      const uint32_t kind = m->remote[r].kind;
      if (r == rank) {
        m->mapped[r] = data;
      } else if (kind == static_cast<uint32_t>(MrKind::CUDA_IPC) || kind == static_cast<uint32_t>(MrKind::CUDA_VMM)) {
        void* p = nullptr;
        if (IpcMapper::open_now(m->remote[r].ipc_handle, kind == static_cast<uint32_t>(MrKind::CUDA_VMM), &p, &m->mapped_bytes[r]) == 0)
          m->mapped[r] = static_cast<char*>(p) + (m->remote[r].addr - m->remote[r].key);
      }
    }
  }
  if (type == NCCL_PTR_CUDA) {
    int direct = 0;
    for (int r = 0; r < nranks; ++r) direct += (r != rank && m->mapped[r]) ? 1 : 0;
    NET_INFO(NCCL_NET, "GIN registration of %zu bytes of device memory: %d of %d peers mapped directly (%s)", size, direct,
             nranks - 1, mine.kind == static_cast<uint32_t>(MrKind::CUDA_VMM) ? "exported as a descriptor"
                         : mine.kind == static_cast<uint32_t>(MrKind::CUDA_IPC) ? "legacy IPC handle" : "no handle: peers send fragments");
  }
  mrs_.push_back(m);
  B200NET_TRACE_EVENT(GinRegMr, dev, comm_id, 0, size, m);
  *out = m;
  return 0;
}

int CollComm::dereg_mr_sym(SymmMr* mr) {
  std::lock_guard<std::recursive_mutex> g(lock);
  if (!mr) return 0;
  if (--mr->refcnt > 0) return 0;
  for (auto it = mrs_.begin(); it != mrs_.end(); ++it)
    if (*it == mr) {
      mrs_.erase(it);
      break;
    }
  if (mr->type == NCCL_PTR_CUDA)
    for (int r = 0; r < nranks; ++r)
      if (r != rank && mr->mapped[r])
        IpcMapper::close_now(static_cast<char*>(mr->mapped[r]) - (mr->remote[r].addr - mr->remote[r].key),
                             mr->remote[r].kind == static_cast<uint32_t>(MrKind::CUDA_VMM), mr->mapped_bytes[r]);
  if (mr->export_fd >= 0) ::close(mr->export_fd);
  if (mr->gpu_handle_block) cuda::mem_free(mr->gpu_handle_block);
  B200NET_TRACE_EVENT(GinDeregMr, dev, comm_id, 0, mr->size, mr);
  delete mr;
  return 0;
}

int CollComm::send_ack(uint32_t peer_rank) {
  PeerState& p = peers_[peer_rank];
  AckMsg a{p.comm_id, static_cast<uint32_t>(rank), p.rx_applied};
  const int rc = fab_.send(p.map, DgramType::GIN_ACK, 0, &a, sizeof(a));
  if (rc == 0) {
    p.rx_acked = p.rx_applied;
    B200NET_TRACE_EVENT(GinAckSend, dev, comm_id, static_cast<uint32_t>(a.acked_seq), 0, this);
  }
  return rc;
}

int CollComm::apply_signal(const MetadataMsg& m) {
  if (m.signal_op != NCCL_NET_SIGNAL_OP_INC && m.signal_op != NCCL_NET_SIGNAL_OP_ADD) return -EINVAL;
  // bounds: the word must lie inside one of this rank's registrations
  bool inside = false;
  for (SymmMr* mr : mrs_) {
    const uint64_t b = reinterpret_cast<uint64_t>(mr->base);
    if (m.signal_addr >= b && m.signal_addr + 8 <= b + mr->size) inside = true;
  }
  if (!inside) {
    NET_WARN("signal address %llx outside every registration: dropped", static_cast<unsigned long long>(m.signal_addr));
    error_ = true;
    return -EFAULT;
  }
  const uint64_t add = m.signal_op == NCCL_NET_SIGNAL_OP_INC ? 1 : m.signal_value;
  if (m.signal_is_device) {
    if (!DeviceSignalWorker::instance().submit(SignalWork{m.signal_addr, add, m.src_rank, 0})) return -EAGAIN;
  } else {
    __atomic_fetch_add(reinterpret_cast<uint64_t*>(m.signal_addr), add, __ATOMIC_RELEASE);
  }
  B200NET_TRACE_EVENT(GinSignalDeliver, dev, comm_id, static_cast<uint32_t>(m.seq), add, this);
  PluginStats::bump(PluginStats::get().gin_signals_applied);
  return 0;
}

void CollComm::handle_dgram(const DgramHdr& h, const void* payload) {
  if (h.type == static_cast<uint16_t>(DgramType::GIN_METADATA)) {
    const auto* m = static_cast<const MetadataMsg*>(payload);
    if (m->comm_id != comm_id || m->src_rank >= static_cast<uint32_t>(nranks)) return;
    B200NET_TRACE_EVENT(GinMetadataRecv, dev, comm_id, static_cast<uint32_t>(m->seq), 0, this);
    PeerState& p = peers_[m->src_rank];
    if (m->signal_addr) {
      if (apply_signal(*m) == -EAGAIN) deferred_signals_.push_back(*m);
    }
    if (m->seq > p.rx_applied) p.rx_applied = m->seq;
    const uint32_t interval = static_cast<uint32_t>(params().gin_ack_interval.get());
    if (p.rx_applied - p.rx_acked >= interval) send_ack(m->src_rank);
  } else if (h.type == GIN_DEVICE_FRAG) {
    const auto* fh = static_cast<const GinDeviceFragHdr*>(payload);
    if (fh->comm_id != comm_id || h.len < sizeof(*fh) + fh->len) return;
    // only into device memory registered with this communicator
    bool inside = false;
    for (SymmMr* mr : mrs_) {
      const uint64_t b = reinterpret_cast<uint64_t>(mr->base);
      if (mr->type == NCCL_PTR_CUDA && fh->addr >= b && fh->addr + fh->len <= b + mr->size) inside = true;
    }
    static thread_local cuda::Stream st = nullptr;
    if (!inside || (!st && cuda::stream_create(&st) != 0) ||
        cuda::memcpy_async(reinterpret_cast<void*>(fh->addr), static_cast<const char*>(payload) + sizeof(*fh), fh->len, st) != 0 ||
        cuda::stream_synchronize(st) != 0) {   // the ring cell is recycled on return
      NET_WARN("GIN: a fragment for device address %llx (%u bytes) could not be applied", static_cast<unsigned long long>(fh->addr),
               fh->len);
      error_ = true;
    }
  } else if (h.type == static_cast<uint16_t>(DgramType::GIN_ACK)) {
    const auto* a = static_cast<const AckMsg*>(payload);
    if (a->comm_id != comm_id || a->src_rank >= static_cast<uint32_t>(nranks)) return;
    PeerState& p = peers_[a->src_rank];
    if (a->acked_seq > p.tx_acked) p.tx_acked = a->acked_seq;
    B200NET_TRACE_EVENT(GinAckRecv, dev, comm_id, static_cast<uint32_t>(a->acked_seq), 0, this);
  } else if (h.type == static_cast<uint16_t>(DgramType::READ_REQ)) {
    const auto* r = static_cast<const ReadReqMsg*>(payload);
    if (r->comm_id != comm_id || r->src_rank >= static_cast<uint32_t>(nranks)) return;
    read_services_.push_back(ReadService{*r, 0, false, {}});
    PluginStats::bump(PluginStats::get().gin_reads_served);
  } else if (h.type == static_cast<uint16_t>(DgramType::READ_RESP)) {
    const auto* r = static_cast<const ReadRespMsg*>(payload);
    auto it = reads_in_flight_.find(r->req_id);
    if (it != reads_in_flight_.end()) {
      int status = r->status == 0 ? 1 : r->status;
      auto landing = read_landings_.find(r->req_id);
      if (landing != read_landings_.end()) {
        if (status == 1 && !landing->second.host.empty()) {
          static thread_local cuda::Stream st = nullptr;
          if ((!st && cuda::stream_create(&st) != 0) ||
              cuda::memcpy_async(landing->second.device_dst, landing->second.host.data(), landing->second.host.size(), st) != 0 ||
              cuda::stream_synchronize(st) != 0)
            status = -EIO;
        }
        read_landings_.erase(landing);
      }
      B200NET_TRACE_EVENT(GinGetEnd, dev, comm_id, 0, 0, it->second.get());
      it->second->store(status);
      reads_in_flight_.erase(it);
    }
  }
}

// Serve reads requested by peers that cannot reach this rank's memory directly: write the bytes
// into the requester's buffer, then confirm (ordered behind the fragments).
int CollComm::serve_reads() {
  while (!read_services_.empty()) {
    ReadService& sv = read_services_.front();
    PeerState& p = peers_[sv.req.src_rank];
    int status = 0;
    bool inside = false, on_device = false;
    for (SymmMr* mr : mrs_) {
      const uint64_t b = reinterpret_cast<uint64_t>(mr->base);
      if (sv.req.addr >= b && sv.req.addr + sv.req.len <= b + mr->size) {
        inside = true;
        on_device = mr->type == NCCL_PTR_CUDA;
      }
    }
    if (!inside) status = -EFAULT;
    if (!status && on_device && sv.bounce.empty() && sv.req.len) {
      // the requester cannot map this device memory: fetch it once, then write it back like host memory
      static thread_local cuda::Stream st = nullptr;
      sv.bounce.resize(sv.req.len);
      if ((!st && cuda::stream_create(&st) != 0) ||
          cuda::memcpy_async(sv.bounce.data(), reinterpret_cast<const void*>(sv.req.addr), sv.req.len, st) != 0 ||
          cuda::stream_synchronize(st) != 0)
        status = -EIO;
    }
    if (!status && !sv.data_done) {
      const void* from = on_device ? static_cast<const void*>(sv.bounce.data()) : reinterpret_cast<const void*>(sv.req.addr);
      const int rc = fab_.write_host(p.map, sv.req.reply_addr, from, sv.req.len, &sv.done);
      if (rc == -EAGAIN) return 0;
      if (rc != 0) status = rc;
      sv.data_done = true;
    }
    ReadRespMsg resp{p.comm_id, static_cast<uint32_t>(rank), sv.req.req_id, status, 0};
    const int rc = fab_.send(p.map, DgramType::READ_RESP, fab_.writes_are_staged(p.map) ? DGRAM_FLAG_ORDER_AFTER_FRAGS : 0,
                             &resp, sizeof(resp));
    if (rc == -EAGAIN) return 0;
    read_services_.pop_front();
  }
  return 0;
}

// Retire the operations towards one peer strictly in order: an operation's metadata (which carries
// its signal, and advances the peer's applied count) goes out only after its data has landed and
// after every earlier operation's metadata.
int CollComm::retire(PeerState& p, uint32_t peer_rank) {
  auto finish = [&](int status) {   // the front operation is over: publish its status, close its range
    PendingOp& op = p.ops.front();
    if (status < 0) error_ = true;
    if (op.has_signal) B200NET_TRACE_EVENT(GinPutSignalEnd, dev, comm_id, static_cast<uint32_t>(op.seq), op.len, op.status.get());
    else B200NET_TRACE_EVENT(GinPutEnd, dev, comm_id, static_cast<uint32_t>(op.seq), op.len, op.status.get());
    op.status->store(status);
    p.ops.pop_front();
  };
  while (!p.ops.empty()) {
    PendingOp& op = p.ops.front();
    if (!op.data_done) {
      if (op.kslot >= 0) {
        NetKernels* nk = NetKernels::get();
        const int ks = nk ? nk->status(op.kslot) : -EIO;
        if (ks == 0) return 0;
        if (nk) nk->release(op.kslot);
        op.kslot = -1;
        if (ks < 0) {
          finish(-EIO);
          continue;
        }
        op.data_done = true;
      } else if (op.event) {
        const int q = cuda::event_query(op.event);
        if (q < 0) {
          finish(-EIO);
          continue;
        }
        if (q == 1) return 0;
        cuda::event_destroy(op.event);
        op.event = nullptr;
        op.data_done = true;
      } else if (op.len && op.dev_frags) {
        const size_t chunk = FAB_LARGE_CELL - sizeof(GinDeviceFragHdr) - 64;
        int rc = 0;
        while (op.done < op.len) {
          const size_t nbytes = std::min(chunk, op.len - op.done);
          GinDeviceFragHdr fh{p.comm_id, static_cast<uint32_t>(nbytes), op.remote_addr + op.done};
          rc = fab_.send(p.map, static_cast<DgramType>(GIN_DEVICE_FRAG), DGRAM_FLAG_ORDER_AFTER_FRAGS, &fh, sizeof(fh),
                         static_cast<const char*>(op.local) + op.done, nbytes);
          if (rc != 0) break;
          op.done += nbytes;
        }
        if (rc == -EAGAIN) return 0;
        if (rc != 0) {
          finish(rc);
          continue;
        }
        op.staged = true;   // the metadata must queue behind the fragments
        op.data_done = true;
      } else if (op.len) {
        const int rc = fab_.write_host(p.map, op.remote_addr, op.local, op.len, &op.done);
        if (rc == -EAGAIN) return 0;
        if (rc != 0) {
          finish(rc);
          continue;
        }
        op.staged = fab_.writes_are_staged(p.map);
        op.data_done = true;
      } else {
        op.data_done = true;
      }
    }
    if (!op.signal_sent) {
      const int rc = fab_.send(p.map, DgramType::GIN_METADATA, op.staged ? DGRAM_FLAG_ORDER_AFTER_FRAGS : 0, &op.meta,
                               sizeof(op.meta));
      if (rc == -EAGAIN) return 0;
      if (rc != 0) {
        finish(rc);
        continue;
      }
      op.signal_sent = true;
      B200NET_TRACE_EVENT(GinMetadataSend, dev, comm_id, static_cast<uint32_t>(op.seq), 0, this);
    }
    finish(1);
    (void)peer_rank;
  }
  return 0;
}

int CollComm::progress() {
  std::lock_guard<std::recursive_mutex> g(lock);
  if (const int got = fab_.poll(256, [this](const DgramHdr& h, const void* p) { handle_dgram(h, p); }); got > 0)
    B200NET_TRACE_EVENT(GinProgress, dev, comm_id, 0, static_cast<uint64_t>(got), this);
  while (!deferred_signals_.empty()) {
    if (apply_signal(deferred_signals_.front()) == -EAGAIN) break;
    deferred_signals_.pop_front();
  }
  for (int r = 0; r < nranks; ++r) retire(peers_[r], static_cast<uint32_t>(r));
  serve_reads();
  return 0;
}

int CollComm::iput(uint64_t src_off, SymmMr* src, size_t size, uint64_t dst_off, SymmMr* dst, uint32_t peer_rank,
                   bool with_signal, uint64_t sig_off, SymmMr* sig, uint64_t sig_value, uint32_t sig_op,
                   GinRequest** req) {
  std::lock_guard<std::recursive_mutex> g(lock);
  *req = nullptr;
  if (closing_) return -ESHUTDOWN;
  if (peer_rank >= static_cast<uint32_t>(nranks)) return -EINVAL;
  if (size && (!src || !dst || src_off + size > src->size || dst_off + size > dst->remote[peer_rank].size)) return -EINVAL;
  if (with_signal && (!sig || sig_off + 8 > sig->remote[peer_rank].size)) return -EINVAL;
  progress();
  PeerState& p = peers_[peer_rank];
  if (p.tx_head - p.tx_acked >= GIN_ACK_REQ_THRESHOLD) return 0;  // window full: no request, call again
  PendingOp op;
  op.len = size;
  op.status = std::make_shared<std::atomic<int>>(0);
  op.has_signal = with_signal;
  memset(&op.meta, 0, sizeof(op.meta));
  op.meta.comm_id = p.comm_id;
  op.meta.src_rank = static_cast<uint32_t>(rank);
  if (with_signal) {
    op.meta.signal_addr = sig->remote[peer_rank].addr + sig_off;
    op.meta.signal_value = sig_value;
    op.meta.signal_op = sig_op;
    op.meta.signal_is_device = sig->remote[peer_rank].kind != static_cast<uint32_t>(MrKind::HOST);
  }
  if (size) {
    const char* lsrc = static_cast<const char*>(src->base) + src_off;
    const RemoteMr& rm = dst->remote[peer_rank];
    PluginStats& st_ = PluginStats::get();
    PluginStats::bump(rm.kind == static_cast<uint32_t>(MrKind::HOST) ? st_.gin_bytes_host
                      : dst->mapped[peer_rank]                        ? st_.gin_bytes_direct
                                                                      : st_.gin_bytes_fragments,
                      size);
    if (rm.kind == static_cast<uint32_t>(MrKind::HOST)) {
      if (src->type == NCCL_PTR_CUDA) {
        // the host write path reads its source with the CPU: fetch the device bytes first
        static thread_local cuda::Stream st = nullptr;
        if (!st && cuda::stream_create(&st) != 0) return -EIO;
        op.bounce.resize(size);
        if (cuda::memcpy_async(op.bounce.data(), lsrc, size, st) != 0 || cuda::stream_synchronize(st) != 0) return -EIO;
        op.local = op.bounce.data();
      } else {
        op.local = lsrc;
      }
      op.remote_addr = rm.addr + dst_off;
    } else if (dst->mapped[peer_rank]) {
      // device window mapped here: the plugin's copy kernel writes it (a device source, or a
      // page-locked host source read in place) and sets a completion word; without the kernels, or
      // for a pageable host source, a copy-engine transfer with an event
      char* target = static_cast<char*>(dst->mapped[peer_rank]) + dst_off;
      NetKernels* nk = NetKernels::get();
      const void* ksrc = lsrc;
      void* alias = nullptr;
      if (nk && src->type != NCCL_PTR_CUDA) ksrc = cuda::host_device_alias(lsrc, &alias) == 0 ? alias : nullptr;
      if (!(nk && ksrc && nk->stream() && nk->copy_flag(target, ksrc, size, nk->stream(), 0, &op.kslot, src->type == NCCL_PTR_CUDA) == 0)) {
        op.kslot = -1;
        static thread_local cuda::Stream st = nullptr;
        if (!st && cuda::stream_create(&st) != 0) return -EIO;
        if (cuda::event_create(&op.event) != 0) return -EIO;
        if (cuda::memcpy_async(target, lsrc, size, st) != 0 || cuda::event_record(op.event, st) != 0) {
          cuda::event_destroy(op.event);
          return -EIO;
        }
      }
    } else {
      // a device window that cannot be mapped into this process: fragments through host memory
      if (src->type == NCCL_PTR_CUDA) {
        static thread_local cuda::Stream st = nullptr;
        if (!st && cuda::stream_create(&st) != 0) return -EIO;
        op.bounce.resize(size);
        if (cuda::memcpy_async(op.bounce.data(), lsrc, size, st) != 0 || cuda::stream_synchronize(st) != 0) return -EIO;
        op.local = op.bounce.data();
      } else {
        op.local = lsrc;
      }
      op.remote_addr = rm.addr + dst_off;
      op.dev_frags = true;
    }
  }
  PluginStats::bump(PluginStats::get().gin_puts);
  auto status = op.status;
  // the range of a put runs from here to the moment its metadata has left (or it has failed); the
  // status word is what tells two puts with equal per-peer sequence numbers apart
  // the sequence number is taken only now: a put that failed above must not leave a hole in the
  // numbers the peer acknowledges in order
  op.seq = ++p.tx_head;
  op.meta.seq = op.seq;
  if (with_signal) B200NET_TRACE_EVENT(GinPutSignalBegin, dev, comm_id, static_cast<uint32_t>(op.seq), size, status.get());
  else B200NET_TRACE_EVENT(GinPutBegin, dev, comm_id, static_cast<uint32_t>(op.seq), size, status.get());
  p.ops.push_back(std::move(op));
  retire(p, peer_rank);
  *req = new StatusRequest(this, status);
  return 0;
}

int CollComm::iget(uint64_t remote_off, SymmMr* remote, size_t size, uint64_t local_off, SymmMr* local,
                   uint32_t peer_rank, GinRequest** req) {
  std::lock_guard<std::recursive_mutex> g(lock);
  *req = nullptr;
  if (peer_rank >= static_cast<uint32_t>(nranks) || !remote || !local) return -EINVAL;
  if (remote_off + size > remote->remote[peer_rank].size || local_off + size > local->size) return -EINVAL;
  progress();
  PluginStats::bump(PluginStats::get().gin_gets);
  auto status = std::make_shared<std::atomic<int>>(0);
  // the range of a get ends when this call returns, unless the read was handed to the owner: then
  // it ends when the response arrives
  struct GetRange {
    CollComm* c; size_t size; const void* key; bool armed;
    ~GetRange() { if (armed) B200NET_TRACE_EVENT(GinGetEnd, c->dev, c->comm_id, 0, size, key); }
  } range{this, size, status.get(), true};
  B200NET_TRACE_EVENT(GinGetBegin, dev, comm_id, 0, size, status.get());
  char* ldst = static_cast<char*>(local->base) + local_off;
  const RemoteMr& rm = remote->remote[peer_rank];
  int rc = 0;
  if (rm.kind == static_cast<uint32_t>(MrKind::HOST)) {
    // host bytes are read by the CPU; a device destination gets them through a host landing buffer
    const bool to_device = local->type == NCCL_PTR_CUDA;
    std::vector<uint8_t> landing(to_device ? size : 0);
    char* host_dst = to_device ? reinterpret_cast<char*>(landing.data()) : ldst;
    rc = fab_.read_host(peers_[peer_rank].map, rm.addr + remote_off, host_dst, size);
    if (rc == -ENOTSUP) {
      // no direct access to the peer's memory: ask it to write the bytes here
      PeerState& p = peers_[peer_rank];
      ReadReqMsg rq{p.comm_id, static_cast<uint32_t>(rank), next_read_id_++, rm.addr + remote_off, size,
                    reinterpret_cast<uint64_t>(host_dst)};
      if (to_device) {
        // the landing buffer must keep its address until the response: park it first
        ReadLanding& l = read_landings_[rq.req_id];
        l.host = std::move(landing);
        l.device_dst = ldst;
        rq.reply_addr = reinterpret_cast<uint64_t>(l.host.data());
      }
      rc = fab_.send(p.map, DgramType::READ_REQ, 0, &rq, sizeof(rq));
      if (rc != 0) read_landings_.erase(rq.req_id);
      if (rc == -EAGAIN) return 0;  // no request: call again
      if (rc != 0) return rc;
      reads_in_flight_[rq.req_id] = status;
      range.armed = false;
      *req = new StatusRequest(this, status);
      return 0;
    }
    if (rc == 0 && to_device && size) {
      static thread_local cuda::Stream st = nullptr;
      if (!st && cuda::stream_create(&st) != 0) return -EIO;
      rc = cuda::memcpy_async(ldst, landing.data(), size, st);
      if (rc == 0) rc = cuda::stream_synchronize(st);
    }
  } else if (remote->mapped[peer_rank]) {
    static thread_local cuda::Stream st = nullptr;
    if (!st && cuda::stream_create(&st) != 0) return -EIO;
    rc = cuda::memcpy_async(ldst, static_cast<char*>(remote->mapped[peer_rank]) + remote_off, size, st);
    if (rc == 0) rc = cuda::stream_synchronize(st);
  } else {
    // device memory of the peer that cannot be mapped here: the owner reads it and writes it back
    const bool to_device = local->type == NCCL_PTR_CUDA;
    PeerState& p = peers_[peer_rank];
    ReadReqMsg rq{p.comm_id, static_cast<uint32_t>(rank), next_read_id_++, rm.addr + remote_off, size,
                  reinterpret_cast<uint64_t>(ldst)};
    if (to_device) {
      ReadLanding& l = read_landings_[rq.req_id];
      l.host.resize(size);
      l.device_dst = ldst;
      rq.reply_addr = reinterpret_cast<uint64_t>(l.host.data());
    }
    rc = fab_.send(p.map, DgramType::READ_REQ, 0, &rq, sizeof(rq));
    if (rc != 0) read_landings_.erase(rq.req_id);
    if (rc == -EAGAIN) return 0;  // no request: call again
    if (rc != 0) return rc;
    reads_in_flight_[rq.req_id] = status;
    range.armed = false;
    *req = new StatusRequest(this, status);
    return 0;
  }
  if (rc != 0) return rc;
  status->store(1);
  *req = new StatusRequest(this, status);
  return 0;
}

// Everything this rank received so far is visible to its GPU: data arrived through coherent
// NVLink / host writes and signals are applied after the data, so a fence plus the drain of the
// device-signal worker is all a flush has to do.
int CollComm::iflush(GinRequest** req) {
  std::lock_guard<std::recursive_mutex> g(lock);
  progress();
  B200NET_TRACE_EVENT(GinFlushBegin, dev, comm_id, 0, 0, nullptr);
  std::atomic_thread_fence(std::memory_order_acq_rel);
  if (cuda::available()) DeviceSignalWorker::instance().drain();
  auto status = std::make_shared<std::atomic<int>>(1);
  B200NET_TRACE_EVENT(GinFlushEnd, dev, comm_id, 0, 0, nullptr);
  *req = new StatusRequest(this, status);
  return 0;
}

int CollComm::create_context(int n_signals, int n_counters, int n_contexts, bool kernel_initiated, GinContext** out) {
  std::lock_guard<std::recursive_mutex> g(lock);
  if (n_signals < 0 || n_counters < 0 || n_contexts < 1 || n_contexts > GIN_MAX_CONTEXTS ||
      n_signals > GIN_MAX_SIGNALS_PER_CONTEXT || n_counters > GIN_MAX_SIGNALS_PER_CONTEXT)
    return -EINVAL;
  auto* c = new GinContext();
  c->comm = this;
  c->n_signals = n_signals;
  c->n_counters = n_counters;
  c->n_contexts = n_contexts;
  c->kernel_initiated = kernel_initiated;
  c->net_dev_handle.netDeviceType = kernel_initiated ? NCCL_NET_DEVICE_GIN_GDAKI : NCCL_NET_DEVICE_GIN_PROXY;
  c->net_dev_handle.netDeviceVersion = 1;
  c->net_dev_handle.needsProxyProgress = kernel_initiated ? 0 : 1;
  if (kernel_initiated) {
    // Ranks may ask for different counts: size the pad for the maximum so every rank's layout agrees.
    std::vector<int32_t> counts(static_cast<size_t>(2 * nranks), 0);
    counts[2 * rank] = n_signals;
    counts[2 * rank + 1] = n_counters;
    int rc = all_gather(counts.data(), 2 * sizeof(int32_t));
    if (rc) {
      delete c;
      return rc;
    }
    int max_sig = 0, max_cnt = 0;
    for (int r = 0; r < nranks; ++r) {
      max_sig = std::max(max_sig, counts[2 * r]);
      max_cnt = std::max(max_cnt, counts[2 * r + 1]);
    }
    if (nranks > b200::GIN_MAX_RANKS || max_sig > b200::GIN_MAX_SIGNALS || max_cnt > b200::GIN_MAX_COUNTERS) {
      NET_WARN("GIN: a kernel-initiated context serves at most %d ranks, %d signals and %d counters", b200::GIN_MAX_RANKS,
               b200::GIN_MAX_SIGNALS, b200::GIN_MAX_COUNTERS);
      delete c;
      return -EINVAL;
    }
    // The pad has the layout of b200net/gin_dev_handle.h: barrier flags, signal words, reset
    // offsets, counters and the status word at fixed offsets, the same on every rank.
    const size_t pad_bytes = b200::GIN_PAD_BYTES;
    if (!cuda::available() || cuda::mem_alloc(&c->dev_pad, pad_bytes) != 0) {   // zero-filled
      delete c;
      return -ENOMEM;
    }
    // exchange the pads' IPC handles in ONE all-gather and map every peer's pad
    struct PadRec { uint8_t ipc[64]; uint64_t bytes; };
    std::vector<PadRec> pads(static_cast<size_t>(nranks));
    memset(pads.data(), 0, pads.size() * sizeof(PadRec));
    pads[rank].bytes = pad_bytes;
    rc = cuda::ipc_get_handle(c->dev_pad, pads[rank].ipc);
    if (rc == 0) rc = all_gather(pads.data(), sizeof(PadRec));
    if (rc) {
      cuda::mem_free(c->dev_pad);
      delete c;
      return rc;
    }
    c->peer_pads.assign(static_cast<size_t>(nranks), nullptr);
    for (int r = 0; r < nranks; ++r) {
      if (r == rank) c->peer_pads[r] = c->dev_pad;
      else if (cuda::ipc_open(pads[r].ipc, &c->peer_pads[r]) != 0) c->has_error = true;
    }
    if (c->has_error) {
      // kernels would store through a null pad address: no context rather than a broken one
      NET_WARN("GIN: a peer's signal pad cannot be mapped into this process; kernel-initiated mode is not available");
      for (int r = 0; r < nranks; ++r)
        if (r != rank && c->peer_pads[r]) cuda::ipc_close(c->peer_pads[r]);
      cuda::mem_free(c->dev_pad);
      delete c;
      return -EIO;
    }
    // the device-visible handle: exactly the structure the device API takes. Windows are not part
    // of a context: a kernel reaches registered memory through the GinDevWindow of its registration.
    b200::GinDevHandle h;
    memset(&h, 0, sizeof(h));
    h.rank = rank;
    h.nranks = nranks;
    for (int r = 0; r < nranks; ++r) h.pad[r] = static_cast<uint8_t*>(c->peer_pads[r]);
    h.status = reinterpret_cast<int*>(static_cast<uint8_t*>(c->dev_pad) + b200::GIN_PAD_STATUS_OFF);
    h.wait_limit_ns = params().device_wait_limit_ms.get() * 1000000ull;
    if (cuda::mem_alloc(&c->dev_handle_gpu, sizeof(h)) != 0) {
      for (int r = 0; r < nranks; ++r)
        if (r != rank && c->peer_pads[r]) cuda::ipc_close(c->peer_pads[r]);
      cuda::mem_free(c->dev_pad);
      delete c;
      return -ENOMEM;
    }
    cuda::Stream st = nullptr;
    cuda::stream_create(&st);
    cuda::memcpy_async(c->dev_handle_gpu, &h, sizeof(h), st);
    cuda::stream_synchronize(st);
    cuda::stream_destroy(st);
    c->n_signals = max_sig;
    c->n_counters = max_cnt;
    c->net_dev_handle.handle = c->dev_handle_gpu;
    c->net_dev_handle.size = sizeof(h);
    NET_INFO(NCCL_INIT | NCCL_NET, "GIN context ready: %d ranks, %d signals, %d counters, %d contexts (kernel-initiated)",
             nranks, max_sig, max_cnt, n_contexts);
  }
  contexts_.push_back(c);
  *out = c;
  return 0;
}

int CollComm::destroy_context(GinContext* ctx) {
  std::lock_guard<std::recursive_mutex> g(lock);
  for (auto it = contexts_.begin(); it != contexts_.end(); ++it) {
    if (*it != ctx) continue;
    contexts_.erase(it);
    if (ctx->kernel_initiated) {
      for (int r = 0; r < nranks; ++r)
        if (r != rank && ctx->peer_pads[r]) cuda::ipc_close(ctx->peer_pads[r]);
      if (ctx->dev_handle_gpu) cuda::mem_free(ctx->dev_handle_gpu);
      if (ctx->dev_pad) cuda::mem_free(ctx->dev_pad);
    }
    delete ctx;
    return 0;
  }
  return -ENOENT;
}

int CollComm::close() {
  {
    std::lock_guard<std::recursive_mutex> g(lock);
    closing_ = true;
  }
  // phase 1: everything issued must retire, and every peer must learn how far we applied its ops
  const auto t0 = Clock::now();
  for (;;) {
    progress();
    std::lock_guard<std::recursive_mutex> g(lock);
    bool busy = false;
    for (int r = 0; r < nranks; ++r) {
      if (!peers_[r].ops.empty()) busy = true;
      if (peers_[r].map && peers_[r].rx_applied != peers_[r].rx_acked) send_ack(static_cast<uint32_t>(r));
    }
    if (!busy && deferred_signals_.empty()) break;
    if (expired(t0)) {
      NET_WARN("GIN close: operations still pending after the deadline");
      break;
    }
  }
  // phase 2: a ring barrier so that no rank tears its endpoint down while a peer may still write
  if (nranks > 1 && ring_send_ && ring_recv_) {
    std::vector<uint8_t> tok(static_cast<size_t>(nranks), 0);
    all_gather(tok.data(), 1);
  }
  std::lock_guard<std::recursive_mutex> g(lock);
  // contexts NCCL never destroyed are swept here
  while (!contexts_.empty()) destroy_context(contexts_.back());
  if (ring_send_) api::close_send(ring_send_);
  if (ring_recv_) api::close_recv(ring_recv_);
  ring_send_ = ring_recv_ = nullptr;
  B200NET_TRACE_EVENT(GinClose, dev, comm_id, 0, 0, this);
  return 0;
}

}  // namespace b200net::gin
