// RDMA-style transport: receiver-driven rendezvous through a control mailbox, multi-rail striped
// writes with completion notifications, an eager path for small messages, grouped receives, a
// retry queue for back-pressured posts, close messages and endpoint abort
// (reference: src/nccl_ofi_rdma.cpp — send() :5646-5877, recv() :3545-3746, test() :2234-2307,
//  the completion loop :1485-1568, pending-request retries :1376-1453, close :3895-4304).
//
// The "wire" is the shared-memory fabric for host buffers and CUDA IPC / VMM mappings of the peer's
// device buffers, written by the plugin's own copy kernel (or the copy engine) on per-rail streams;
// the protocol state machine is independent of it.
//
// Nothing on the send / receive / test path waits for the device: a copy is posted, the request
// stays pending, and its completion word or event is polled from test(). The thread that drives
// this code is NCCL's proxy, and NCCL's kernel on the same device waits for the proxy, so a driver
// call that waits for the device could wait for ever. Requests, eager staging slots and events
// come from pools that belong to the endpoint and are sized when it is created
// (reference: the request, control, eager and flush freelists, src/nccl_ofi_rdma.cpp:4762-4978, and
// the receive-buffer pools :1795-1919).
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
#include <new>
#include <set>
#include <vector>

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
  int rail = 0;
  size_t offset = 0, len = 0, done = 0;
  cuda::Event event = nullptr;   // non-null while a copy-engine transfer is in flight (from the endpoint's pool)
  bool posted = false, complete = false, notified = false;
  int kslot = -1;      // completion slot of a copy-kernel transfer in flight
  uint64_t t_launch_ns = 0;   // when its launch call returned (latency histograms only)
  std::shared_ptr<std::atomic<int>> job;  // status of a stripe handed to a host copy worker
};

// Where a send writes: the fields of the control entry it was matched to.
struct SendTarget {
  uint64_t buff_addr = 0, mr_key = 0, buff_len = 0;
  uint16_t flags = 0;
};

class RdmaSendReq : public Request {
 public:
  int test(int* done, int* sizes) override;
  // A stripe still held by a copy worker reads this request's source buffer: wait for it.
  ~RdmaSendReq() override {
    for (int i = 0; i < nstripes; ++i)
      while (stripes[i].job && stripes[i].job->load(std::memory_order_acquire) == 0) sched_yield();
  }
  FreelistEntry* fl = nullptr;   // the pool entry this object lives in
  RdmaSendComm* comm = nullptr;
  void* data = nullptr;
  size_t size = 0;
  int tag = 0;
  ReqState state = ReqState::CREATED;
  bool eager = false;       // sent eagerly, waiting to be bound to a control entry
  uint16_t seq = 0;
  uint8_t recv_idx = 0;
  SendTarget target;
  Stripe stripes[MAX_NUM_RAILS];
  int nstripes = 0;
  // A device source whose destination is only reachable through host memory is fetched once into
  // `bounce`; the stripes start when the event behind that copy has completed.
  std::vector<uint8_t> bounce;
  cuda::Event bounce_ev = nullptr;
  bool src_dev = false;         // the source is device memory (from its registration, else asked of the driver)
  const char* src_alias = nullptr;  // page-locked host source: where the copy kernel reads it
  bool via_frags = false;       // the target registration has an IPC handle that could not be opened here
  uint64_t serial = 0;          // unique per endpoint; queued retries name the request by it
  // eager sends: the datagram leaves from the communicator's outbox, in eager_seq order, once the
  // payload is in host memory (pack kernel: completion word of `pack_slot`; copy engine: `stage_ev`)
  EagerHdr ehdr{};
  bool dgram_sent = false;
  int pack_slot = -1;
  FreelistEntry* stage = nullptr;
  cuda::Event stage_ev = nullptr;
  uint64_t t_outbox_ns = 0;
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
  FreelistEntry* fl = nullptr;
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
  FreelistEntry* fl = nullptr;
  RdmaEndpoint* ep;
};

struct EagerRx {  // an eager message that arrived before (or without) a matching posted receive
  EagerHdr hdr;
  FreelistEntry* slot;   // staging slot holding the payload (null for an empty message)
};

// Receiver-side work that has to wait for a copy on the endpoint's receive stream, kept in issue
// order: the stream runs its copies in order, so the queue is retired from the front.
struct Deferred {
  enum Kind : uint8_t { FRAG_COPY, EAGER_COPY, WRITE_COMPLETION } kind;
  cuda::Event ev = nullptr;        // copy-engine copy: its event. No event and no kernel slot: ready as soon
                                   // as everything before it has retired
  int kslot = -1;                  // copy-kernel copy: its completion slot
  FreelistEntry* slot = nullptr;   // staging slot to give back
  uint32_t comm_id = 0;            // EAGER_COPY: the receive it completes
  uint16_t seq = 0;
  uint8_t idx = 0;
  WriteCompletion wc{};            // WRITE_COMPLETION: applied once the fragments before it have landed
};

// A typed view of a Freelist: objects are constructed when taken and destroyed when given back.
template <typename T>
class ObjPool {
 public:
  ObjPool(const char* name, size_t initial, size_t grow, size_t max = 0)
      : fl_(Freelist::Options{sizeof(T), initial, grow, max, alignof(T) < 8 ? 8 : alignof(T), 4096, nullptr, nullptr, nullptr, nullptr, name}) {}
  template <typename... A>
  T* take(A&&... a) {
    FreelistEntry* e = fl_.entry_alloc();
    if (!e) return nullptr;
    T* t = new (e->ptr) T(std::forward<A>(a)...);
    t->fl = e;
    return t;
  }
  void give(T* t) {
    FreelistEntry* e = t->fl;
    t->~T();
    fl_.entry_free(e);
  }
  size_t in_use() const { return fl_.in_use(); }

 private:
  Freelist fl_;
};

constexpr size_t STAGE_BYTES = FAB_LARGE_CELL;   // one eager payload or one fragment

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
  void retire_deferred();
  void flush_outboxes();
  void fail_endpoint(const char* why, int rc);
  int ensure_published(MrHandle* mh);
  cuda::Stream rail_stream(int rail);
  // The mapping of a peer's device registration in this process, or nullptr while it does not
  // exist (in progress on the helper thread, or failed). wait: give a first open the grace period.
  void* map_peer_cuda(PeerMapping* peer, const MrTableEntry* e, bool wait = true);
  // Queues the open of every device registration the peer has published so far. Called on set-up
  // paths (a connection completes, a buffer is registered), so that the first send rarely has to.
  void premap_peer(PeerMapping* peer);
  // Loads the plugin's device kernels into the current context, creates the streams, the event
  // pool and the page-locked staging slots. Only called from set-up paths (registration, connect,
  // listen): loading a module, creating a stream or page-locking memory while a collective kernel
  // that waits for this very transport is running can block for ever.
  void prepare_kernels();
  cuda::Event take_event();
  // Queues dst[0,n) = the staging slot's bytes on the receive stream: the copy kernel reading the
  // page-locked slot in place when the kernels are loaded, else the copy engine. Fills d->kslot or
  // d->ev. 0 or a negative error.
  int stage_to_device(void* dst, FreelistEntry* slot, size_t n, Deferred* d);
  void give_event(cuda::Event ev) { if (ev) free_events.push_back(ev); }
  Freelist& staging() { return *staging_; }

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
  // Sends whose post met a full ring (-EAGAIN), by serial number, retried strictly in order. A
  // request's address can be handed out again (to another communicator's request) while an old
  // retry for it is still queued; its serial number cannot.
  std::deque<uint64_t> pending;
  std::map<uint64_t, RdmaSendReq*> live_send_reqs;
  uint64_t next_req_serial = 1;
  std::vector<cuda::Stream> streams;
  // (peer pid, IPC handle bytes) -> mapped base. Keyed by the handle, not by the MR key: keys are
  // recycled when a buffer is deregistered, and a new registration under an old key is a
  // different allocation.
  std::map<std::pair<uint32_t, std::array<uint8_t, 64>>, std::shared_ptr<IpcMapJob>> ipc_maps;
  bool warned_ipc = false, noted_ipc_wait = false;
  void note_unmapped(PeerMapping* peer, const MrTableEntry* e);
  std::set<std::pair<MrHandle*, int>> published;
  std::map<MrHandle*, int> export_fds;   // descriptors kept open for peers that import a CUDA_VMM registration
  // pools
  ObjPool<RdmaSendReq> send_reqs{"send requests", 256, 256};
  ObjPool<RdmaRecvReq> recv_reqs{"receive requests", NET_MAX_REQUESTS, NET_MAX_REQUESTS};
  ObjPool<RdmaFlushReq> flush_reqs{"flush requests", 32, 32};
  std::unique_ptr<Freelist> staging_;
  std::vector<cuda::Event> free_events;
  std::deque<Deferred> deferred;
  int outbox_total = 0;        // eager sends of all communicators whose datagram has not left yet
  bool in_progress = false;
  // stall report: when requests are in flight and nothing has moved for STALL_REPORT_MS, the state
  // of every queue goes to the log once (and again after the next sign of life)
  uint64_t last_activity_ns = 0, last_progress_ns = 0;
  bool stall_reported = false;
  void note_activity() {
    last_activity_ns = PluginStats::now_ns();
    stall_reported = false;
  }
  void report_stall();
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
  std::deque<RdmaSendReq*> outbox;   // eager sends whose datagram has not left yet, in eager_seq order
  void flush_outbox();
  void release(RdmaSendReq* r);
  std::unique_ptr<ThresholdScheduler> sched;
  int inflight = 0;
  uint64_t accepted = 0;        // sends that got a request
  uint64_t refused_since = 0;   // send calls since then that found neither a receive nor room for an eager send
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
  void fail_sub(RdmaRecvReq* r, int idx);
  void release(RdmaRecvReq* r);
  RdmaEndpoint* rep() { return static_cast<RdmaEndpoint*>(ep); }

  std::unique_ptr<ShmWindow> mailbox;  // sender's mailbox, mapped
  PeerMapping* peer = nullptr;
  uint16_t next_seq = 0;
  std::unique_ptr<MsgBuff> msgbuff;
  std::list<RdmaRecvReq*> posted;      // incomplete receive groups, oldest first
  std::vector<EagerRx> eager_rx;       // arrived eager messages in eager_seq order (at most a few dozen)
  uint16_t eager_arrived = 0;          // eager messages with a sequence number before this have all arrived
  uint8_t eager_taken[MAILBOX_SLOTS] = {};  // per group: entries matched to eager messages / completed
  int inflight = 0;
  uint32_t nonce = 0;
  bool peer_closed = false;
};

// ------------------------------------------------------------------------------------------ endpoint impl
RdmaEndpoint::RdmaEndpoint(Domain* d, int rails) : Endpoint(d), cm(&fab), num_rails(rails) {
  // Staging slots for eager payloads and fragments. Page-locked when a CUDA context is current at
  // the time a block is added (asynchronous copies from page-locked memory do not pass through the
  // driver's staging buffer); plain memory otherwise, which is all a host-only run needs.
  Freelist::Options o;
  o.entry_size = STAGE_BYTES;
  o.initial_count = 0;
  o.grow_count = 64;
  o.max_count = 2048;
  o.entry_align = 64;
  o.name = "staging slots";
  o.reg = [](void* base, size_t bytes, void** handle) {
    *handle = nullptr;
    cuda::Context ctx = nullptr;
    if (cuda::available() && cuda::ctx_get_current(&ctx) == 0 && ctx && cuda::host_register(base, bytes) == 0) *handle = base;
    return 0;
  };
  o.dereg = [](void* handle) { return handle ? cuda::host_unregister(handle) : 0; };
  staging_ = std::make_unique<Freelist>(std::move(o));
}

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
  // Tear-down may wait for the device: copies that still read staging slots must be over before
  // the slots are unpinned and unmapped.
  for (auto s : streams)
    if (s) cuda::stream_synchronize(s);
  for (Deferred& d : deferred) {
    give_event(d.ev);
    if (d.slot) staging_->entry_free(d.slot);
  }
  deferred.clear();
  for (auto& [k, job] : ipc_maps)
    if (job && job->abandon()) job->close_mapping();
  for (auto& [mh, fd] : export_fds) ::close(fd);
  for (cuda::Event ev : free_events) cuda::event_destroy(ev);
  for (auto s : streams)
    if (s) cuda::stream_destroy(s);
}

void RdmaEndpoint::prepare_kernels() {
  if (kernels_tried || !cuda::available()) return;
  cuda::Context ctx = nullptr;
  if (cuda::ctx_get_current(&ctx) != 0 || !ctx) return;
  kernels = NetKernels::get();
  kernels_tried = true;
  for (int rail = 0; rail < num_rails; ++rail) rail_stream(rail);
  for (int i = 0; i < 128; ++i) {
    cuda::Event ev = nullptr;
    if (cuda::event_create(&ev) == 0) free_events.push_back(ev);
  }
  // the first block of staging slots is page-locked here, not under a running collective
  if (FreelistEntry* e = staging_->entry_alloc()) staging_->entry_free(e);
}

cuda::Event RdmaEndpoint::take_event() {
  if (!free_events.empty()) {
    cuda::Event ev = free_events.back();
    free_events.pop_back();
    return ev;
  }
  cuda::Event ev = nullptr;   // the pool ran dry (more copies in flight than it was sized for)
  return cuda::event_create(&ev) == 0 ? ev : nullptr;
}

int RdmaEndpoint::stage_to_device(void* dst, FreelistEntry* slot, size_t n, Deferred* d) {
  cuda::Stream st = rail_stream(0);
  if (!st) return -EIO;
  void* alias = nullptr;
  if (kernels && slot->mr_handle && cuda::host_device_alias(slot->ptr, &alias) == 0 &&
      kernels->copy_flag(dst, alias, n, st, 1, &d->kslot, false) == 0)
    return 0;
  d->kslot = -1;
  d->ev = take_event();
  if (!d->ev) return -ENOMEM;
  int rc = cuda::memcpy_async(dst, slot->ptr, n, st);
  if (rc == 0) rc = cuda::event_record(d->ev, st);
  if (rc != 0) {
    give_event(d->ev);
    d->ev = nullptr;
  }
  return rc;
}

cuda::Stream RdmaEndpoint::rail_stream(int rail) {
  // with the kernels loaded, everything runs on their one stream (see NetKernels::stream)
  if (kernels && kernels->stream() && params().shared_stream.get()) return kernels->stream();
  if (streams.empty()) streams.assign(static_cast<size_t>(num_rails), nullptr);
  rail %= num_rails;
  if (!streams[rail]) {
    if (domain->device->gpu_ordinal >= 0) cuda::ensure_primary_ctx(domain->device->gpu_ordinal);
    if (cuda::stream_create(&streams[rail]) != 0) return nullptr;
  }
  return streams[rail];
}

void* RdmaEndpoint::map_peer_cuda(PeerMapping* peer, const MrTableEntry* e, bool wait) {
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
  }
  if (!it->second) return nullptr;
  if (wait && it->second->state.load(std::memory_order_acquire) == 0 && !it->second->waited) {
    // once an open has outlasted the grace period the device is evidently busy: later first uses
    // stall the caller only briefly (an open that does not have to wait for the device takes microseconds)
    it->second->waited = true;
    const uint64_t grace = params().ipc_map_wait_us.get();
    IpcMapper::wait(*it->second, noted_ipc_wait ? std::min<uint64_t>(grace, 500) : grace);
  }
  return it->second->state.load(std::memory_order_acquire) == 1 ? it->second->mapped : nullptr;
}

void RdmaEndpoint::premap_peer(PeerMapping* peer) {
  if (!peer || !peer->mr_table || !cuda::available()) return;
  cuda::Context ctx = nullptr;
  if (cuda::ctx_get_current(&ctx) != 0 || !ctx) return;
  for (size_t i = 0; i < FAB_MR_TABLE_SLOTS; ++i) {
    const MrTableEntry* e = &peer->mr_table[i];
    if (reinterpret_cast<const std::atomic<uint64_t>*>(&e->key)->load(std::memory_order_acquire) == 0) continue;
    if (e->kind == static_cast<uint32_t>(MrKind::CUDA_IPC) || e->kind == static_cast<uint32_t>(MrKind::CUDA_VMM)) map_peer_cuda(peer, e, false);
  }
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

// Publishes what a peer needs to write into the registration. For device memory the entry
// describes the ALLOCATION the registration lies in: its base and size as the driver reports them
// and the handle taken from that base. A peer adds (address - base) to what its open of the handle
// returned, which is the driver's contract for a handle; nothing is assumed about what else lies
// in the same page or the same backing block.
int RdmaEndpoint::ensure_published(MrHandle* mh) {
  if (!mh) return 0;
  if (published.count({mh, 0})) return 0;
  static std::atomic<uint64_t> next_serial{1};
  MrTableEntry e;
  memset(&e, 0, sizeof(e));
  e.key = mh->key;
  e.base = reinterpret_cast<uint64_t>(mh->base);
  e.size = mh->size;
  e.kind = static_cast<uint32_t>(mh->kind);
  e.serial = next_serial.fetch_add(1);
  if (mh->kind == MrKind::CUDA_IPC) {
    int dev = 0;
    cuda::pointer_info(mh->base, &dev, nullptr, nullptr, nullptr);
    e.device = static_cast<uint32_t>(dev);
    if (cuda::ipc_get_handle(mh->base, e.ipc_handle) != 0) {
      mh->kind = MrKind::CUDA_STAGED;
      e.kind = static_cast<uint32_t>(MrKind::CUDA_STAGED);
    }
  } else if (mh->kind == MrKind::CUDA_VMM) {
    // memory of the virtual-memory API (NCCL's own buffers are such): peers import the allocation
    // behind the mapped range through a descriptor that this process keeps open for them
    int dev = 0, fd = -1;
    cuda::pointer_info(mh->base, &dev, nullptr, nullptr, nullptr);
    if (cuda::vmm_export_range(mh->base, &fd) == 0) {
      VmmShare sh{VMM_SHARE_MAGIC, fd, static_cast<uint32_t>(getpid()), 0, mh->size, e.serial};
      static_assert(sizeof(sh) <= sizeof(e.ipc_handle), "share record fits the handle bytes");
      memcpy(e.ipc_handle, &sh, sizeof(sh));
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

// Host memory: the handle describes the page-rounded range and is shared by every registration
// inside it (the reference registers page-rounded ranges the same way, src/nccl_ofi_mr.cpp).
// Device memory: the handle describes the allocation that contains the range and is shared by
// registrations of that very allocation only; a range that no single allocation covers (an address
// range backed by several allocations of the virtual-memory API) gets a handle of its own and its
// payloads travel as fragments.
int RdmaEndpoint::reg_mr(void* data, size_t size, int type, MrHandle** out) {
  std::lock_guard<std::recursive_mutex> g(ep_lock);
  if (type != NCCL_PTR_HOST) prepare_kernels();
  void* base = data;
  size_t bytes = size;
  MrKind kind = MrKind::HOST;
  MrCacheKey key = MrCacheKey::from_iovec(data, size);
  if (type == NCCL_PTR_CUDA) {
    void* abase = nullptr;
    size_t asize = 0;
    bool vmm = false;
    if (!cuda::available() || cuda::pointer_info(data, nullptr, &abase, &asize, &vmm) != 0) return -EINVAL;
    const bool covered = static_cast<char*>(abase) <= static_cast<char*>(data) &&
                         static_cast<char*>(data) + size <= static_cast<char*>(abase) + asize;
    if (covered) {
      base = abase;
      bytes = asize;
      kind = vmm ? MrKind::CUDA_VMM : MrKind::CUDA_IPC;
    } else {
      kind = MrKind::CUDA_STAGED;
    }
    key = MrCacheKey::from_allocation(base, bytes);
  } else {
    const uintptr_t lo = round_down<uintptr_t>(reinterpret_cast<uintptr_t>(data), MR_CACHE_PAGE_SIZE);
    const uintptr_t hi = round_up<uintptr_t>(reinterpret_cast<uintptr_t>(data) + (size ? size : 1), MR_CACHE_PAGE_SIZE);
    base = reinterpret_cast<void*>(lo);
    bytes = hi - lo;
  }
  MrCache* cache = domain->mr_cache.get();
  MrHandle* mh = cache ? static_cast<MrHandle*>(cache->lookup(key)) : nullptr;
  if (!mh) {
    const uint64_t id = domain->mr_keys.allocate();
    if (id == IdPool::ID_NONE) return -ENOSPC;
    mh = new MrHandle();
    mh->key = id + 1;
    mh->base = base;
    mh->size = bytes;
    mh->type = type;
    mh->domain = domain;
    mh->kind = kind;
    if (cache) {
      const int rc = cache->insert(key, mh);
      if (rc != 0 && rc != -EEXIST) {
        domain->mr_keys.free_id(id);
        delete mh;
        return rc;
      }
    }
    B200NET_TRACE_EVENT(GinRegMr, domain->device->dev_id, 0, 0, size, mh);
  }
  if (type == NCCL_PTR_CUDA) {
    // The export (IPC handle, descriptor) is a driver call: made here, on a set-up path, so that
    // the first receive does not have to make it under a running collective. Peers that are
    // already connected start mapping what the other side has published so far.
    const int rc = ensure_published(mh);
    if (rc != 0) {
      dereg_mr(mh);
      return rc;
    }
    for (auto& [id, sc] : send_comms) premap_peer(sc->peer);
  }
  *out = mh;
  return 0;
}

int RdmaEndpoint::reg_mr_dmabuf(void* data, size_t size, int type, uint64_t offset, int fd, MrHandle** mh) {
  // On NVLink a peer reaches the memory through a mapping of the allocation, which the virtual
  // address identifies; the descriptor names the same allocation. It is checked, not exported.
  if (fd < 0) return -EINVAL;
  (void)offset;
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

void RdmaEndpoint::fail_endpoint(const char* why, int rc) {
  NET_WARN("%s (%d): endpoint aborted", why, rc);
  PluginStats::bump(PluginStats::get().requests_failed);
  invalidate();
}

void RdmaEndpoint::handle_dgram(const DgramHdr& h, const void* payload) {
  if (cm.handle_dgram(h, payload)) return;
  switch (h.type) {
    case static_cast<uint16_t>(DgramType::WRITE_COMPLETION): {
      const auto* wc = static_cast<const WriteCompletion*>(payload);
      if (!deferred.empty()) {
        // fragments that arrived before this completion are still on their way to the device
        Deferred d;
        d.kind = Deferred::WRITE_COMPLETION;
        d.wc = *wc;
        deferred.push_back(d);
        break;
      }
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
      // A piece of a payload whose sender cannot map this process's device memory. The ring cell is
      // recycled on return, so the bytes move to a staging slot; the copy to the device is queued
      // on the receive stream and the write completion that follows waits for it in `deferred`.
      const auto* fh = static_cast<const DeviceFragHdr*>(payload);
      FreelistEntry* slot = fh->len <= STAGE_BYTES ? staging_->entry_alloc() : nullptr;
      if (slot) {
        memcpy(slot->ptr, static_cast<const char*>(payload) + sizeof(*fh), fh->len);
        Deferred d;
        d.kind = Deferred::FRAG_COPY;
        d.slot = slot;
        const int rc = stage_to_device(reinterpret_cast<void*>(fh->remote_addr), slot, fh->len, &d);
        if (rc != 0) {
          staging_->entry_free(slot);
          fail_endpoint("copy of a fragment to the device failed", rc);
        } else {
          deferred.push_back(d);
        }
      } else {
        // no staging slot left: copy straight from the ring cell and wait for this one copy
        cuda::Stream st = rail_stream(0);
        int rc = st ? cuda::memcpy_async(reinterpret_cast<void*>(fh->remote_addr), static_cast<const char*>(payload) + sizeof(*fh), fh->len, st) : -EIO;
        if (rc == 0) rc = cuda::stream_synchronize(st);
        if (rc != 0) fail_endpoint("copy of a fragment to the device failed", rc);
      }
      break;
    }
    default:
      NET_INFO(NCCL_NET, "unexpected datagram type %u dropped", h.type);
  }
}

void RdmaEndpoint::retire_deferred() {
  while (!deferred.empty()) {
    Deferred& d = deferred.front();
    if (d.kslot >= 0) {
      const int ks = kernels ? kernels->status(d.kslot) : -EIO;
      if (ks == 0) return;
      if (kernels) kernels->release(d.kslot);
      d.kslot = -1;
      if (ks < 0) {
        fail_endpoint("a copy on the receive stream failed", ks);
        for (Deferred& x : deferred) {
          give_event(x.ev);
          if (x.slot) staging_->entry_free(x.slot);
        }
        deferred.clear();
        return;
      }
    }
    if (d.ev) {
      const int q = cuda::event_query(d.ev);
      if (q == 1) return;
      if (q < 0) {
        fail_endpoint("a copy on the receive stream failed", q);
        // drop what was queued: the endpoint refuses every later call
        for (Deferred& x : deferred) {
          give_event(x.ev);
          if (x.slot) staging_->entry_free(x.slot);
        }
        deferred.clear();
        return;
      }
      give_event(d.ev);
    }
    if (d.slot) staging_->entry_free(d.slot);
    const Deferred done = d;
    deferred.pop_front();
    if (done.kind == Deferred::WRITE_COMPLETION) {
      auto it = recv_comms.find(done.wc.remote_comm_id);
      if (it != recv_comms.end()) it->second->on_write_completion(done.wc);
    } else if (done.kind == Deferred::EAGER_COPY) {
      auto it = recv_comms.find(done.comm_id);
      if (it == recv_comms.end()) continue;
      void* elem = nullptr;
      MsgElemType ty;
      MsgStatus st;
      if (it->second->msgbuff->retrieve(done.seq, &elem, &ty, &st) == MsgResult::SUCCESS && ty == MsgElemType::REQ)
        it->second->finish_sub(static_cast<RdmaRecvReq*>(elem), done.idx);
    }
  }
}

int RdmaEndpoint::progress() {
  if (in_progress) return 0;  // re-entered from a handler
  in_progress = true;
  const int budget = params().cq_read_count.get() * 16;
  if (PluginStats::get().histograms_on() && !live_send_reqs.empty()) {
    const uint64_t now = PluginStats::now_ns();
    if (last_progress_ns) PluginStats::get().sample_poll_gap(now - last_progress_ns);
    last_progress_ns = now;
  } else {
    last_progress_ns = 0;
  }
  // traced only when the poll found something: an idle proxy thread polls millions of times
  if (const int got = fab.poll(budget, [this](const DgramHdr& h, const void* p) { handle_dgram(h, p); }); got > 0) {
    B200NET_TRACE_EVENT(ProcessCompletionsRdma, domain->device->dev_id, 0, 0, static_cast<uint64_t>(got), this);
    note_activity();
  }
  if (!deferred.empty()) retire_deferred();
  if (outbox_total > 0) flush_outboxes();
  if (kernels) kernels->poll();   // stripes waiting for company leave when an earlier launch has finished
  // retry queue: strictly in order, stop at the first post that is still back-pressured
  while (!pending.empty()) {
    auto live = live_send_reqs.find(pending.front());
    if (live != live_send_reqs.end() && live->second->state == ReqState::PENDING) {
      RdmaSendReq* r = live->second;
      const int rc = r->comm->post_stripes(r);
      if (rc == -EAGAIN) break;
      if (rc != 0 && rc != -EINPROGRESS) r->state = ReqState::ERROR;
    }
    pending.pop_front();
    B200NET_TRACE_EVENT(PendingQueueRemove, domain->device->dev_id, 0, 0, 0, this);
  }
  if (!stall_reported && last_activity_ns) {
    const uint64_t limit_ms = params().stall_report_ms.get();
    if (limit_ms && PluginStats::now_ns() - last_activity_ns > limit_ms * 1000000ull) report_stall();
  }
  in_progress = false;
  return 0;
}

void RdmaEndpoint::report_stall() {
  size_t posted = 0;
  for (auto& [id, rc] : recv_comms) posted += rc->posted.size();
  if (live_send_reqs.empty() && posted == 0) {   // idle, not stalled
    last_activity_ns = PluginStats::now_ns();
    return;
  }
  stall_reported = true;
  NET_WARN("no progress for %llu ms with %zu sends and %zu receive groups in flight; retry queue %zu, deferred %zu, outbox %d, "
           "ring-full answers %llu",
           static_cast<unsigned long long>(params().stall_report_ms.get()), live_send_reqs.size(), posted, pending.size(),
           deferred.size(), outbox_total, static_cast<unsigned long long>(fab.eagain_count()));
  for (auto& [id, sc] : send_comms) {
    auto* box = static_cast<CtrlMsg*>(sc->mailbox->data());
    const CtrlEntry& cur = box[sc->next_seq % MAILBOX_SLOTS].entries[0];
    NET_WARN("  send comm %u -> %u: %d in flight, %llu sends so far, %llu calls since the last one found no receive; group %u taken %#x "
             "(ready word %#x tag %d len %llu; previous slot %#x, next slot %#x), %zu eager unbound, %zu in the outbox%s",
             id, sc->remote_comm_id, sc->inflight, static_cast<unsigned long long>(sc->accepted),
             static_cast<unsigned long long>(sc->refused_since), sc->next_seq, sc->consumed_mask, cur.ready.load(), cur.tag,
             static_cast<unsigned long long>(cur.buff_len), box[(sc->next_seq + MAILBOX_SLOTS - 1) % MAILBOX_SLOTS].entries[0].ready.load(),
             box[(sc->next_seq + 1) % MAILBOX_SLOTS].entries[0].ready.load(), sc->eager_queue.size(), sc->outbox.size(),
             sc->peer_closed ? ", peer closed" : "");
  }
  int shown = 0;
  for (auto& [serial, r] : live_send_reqs) {
    if (++shown > 8) break;
    char per_stripe[MAX_NUM_RAILS * 24 + 8] = "";
    size_t at = 0;
    for (int i = 0; i < r->nstripes && at + 24 < sizeof(per_stripe); ++i) {
      const Stripe& st = r->stripes[i];
      at += static_cast<size_t>(snprintf(per_stripe + at, sizeof(per_stripe) - at, " [rail %d %zuK %s]", st.rail, st.len >> 10,
                                         st.notified ? "done" : st.complete ? "copied" : st.kslot >= 0 ? "kernel" : st.event ? "engine" : st.posted ? "posted" : "new"));
    }
    NET_WARN("    send %llu on comm %u: %zu bytes tag %d state %d %s seq %u;%s%s%s", static_cast<unsigned long long>(serial),
             r->comm->local_comm_id, r->size, r->tag, static_cast<int>(r->state),
             r->eager ? (r->dgram_sent ? "eager, sent" : "eager, in the outbox") : "write", r->seq, per_stripe,
             r->via_frags ? ", as fragments" : "", r->bounce_ev ? ", source still being fetched" : "");
  }
  for (auto& [id, rc] : recv_comms) {
    if (rc->posted.empty() && rc->eager_rx.empty()) continue;
    const RdmaRecvReq* oldest = rc->posted.empty() ? nullptr : rc->posted.front();
    NET_WARN("  recv comm %u <- %u: %d in flight, %zu groups posted (oldest seq %u: %d receives, first %zu bytes tag %d, %zu received in "
             "%d of %d segments), next seq %u, %zu eager messages unmatched, eager sequence %u%s",
             id, rc->remote_comm_id, rc->inflight, rc->posted.size(), oldest ? oldest->seq : 0, oldest ? oldest->n : 0,
             oldest ? oldest->subs[0].cap : 0, oldest ? oldest->subs[0].tag : 0, oldest ? oldest->subs[0].received : 0,
             oldest ? oldest->subs[0].segs_done : 0, oldest ? oldest->subs[0].segs_expected : 0, rc->next_seq, rc->eager_rx.size(),
             rc->eager_arrived, rc->peer_closed ? ", peer closed" : "");
  }
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
  premap_peer(sc->peer);   // whatever the receiver has registered by now is mapped ahead of the first send
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

void RdmaSendComm::release(RdmaSendReq* r) {
  RdmaEndpoint* e = rep();
  --inflight;
  e->live_send_reqs.erase(r->serial);
  // whatever the request still holds goes back to its pool; a copy that is still running keeps
  // its kernel slot (the kernel may yet write the completion word)
  for (int i = 0; i < r->nstripes; ++i) e->give_event(r->stripes[i].event);
  e->give_event(r->bounce_ev);
  e->give_event(r->stage_ev);
  if (r->stage) e->staging().entry_free(r->stage);
  e->send_reqs.give(r);
}

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
    if (r->state == ReqState::PENDING) r->state = ReqState::COMPLETED;
    B200NET_TRACE_EVENT(SendEagerComplete, dev_id, local_comm_id, r->ehdr.eager_seq, r->size, r);
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

// Eager datagrams leave in eager_seq order, each as soon as its payload is in host memory: a host
// source at once, a device source when the pack kernel has set the slot's completion word or the
// copy engine's event has completed. Nothing here waits; a payload that is not ready (or a full
// ring) leaves the rest of the outbox for the next call.
void RdmaSendComm::flush_outbox() {
  RdmaEndpoint* e = rep();
  while (!outbox.empty()) {
    RdmaSendReq* r = outbox.front();
    const void* src = r->data;
    bool failed = false;
    if (r->pack_slot >= 0) {
      if (!e->kernels->eager_done(r->pack_slot)) {
        if (PluginStats::now_ns() - r->t_outbox_ns < 10000000000ull) return;
        NET_WARN("eager pack kernel did not complete within 10 s");   // the slot stays reserved: the kernel may still write it
        r->pack_slot = -1;
        failed = true;
      } else {
        src = e->kernels->eager_slot(r->pack_slot) + 16;
      }
    } else if (r->stage_ev) {
      const int q = cuda::event_query(r->stage_ev);
      if (q == 1) return;
      failed = q < 0;
      src = r->stage->ptr;
    }
    int rc = failed ? -EIO : e->fab.send(peer, DgramType::EAGER, 0, &r->ehdr, sizeof(r->ehdr), src, r->size);
    if (rc == -EAGAIN) return;
    if (r->pack_slot >= 0) e->kernels->eager_release(r->pack_slot);  // the datagram holds a copy
    r->pack_slot = -1;
    if (r->stage) e->staging().entry_free(r->stage);
    r->stage = nullptr;
    e->give_event(r->stage_ev);
    r->stage_ev = nullptr;
    outbox.pop_front();
    --e->outbox_total;
    if (rc != 0) {
      // the receiver waits for this sequence number before it takes later eager messages: the
      // connection cannot continue
      r->state = ReqState::ERROR;
      e->fail_endpoint("an eager payload could not be sent", rc);
      return;
    }
    r->dgram_sent = true;
    e->bytes_eager += r->size;
    PluginStats::bump(PluginStats::get().eager_sends);
  }
}

void RdmaEndpoint::flush_outboxes() {
  for (auto& [id, sc] : send_comms)
    if (!sc->outbox.empty()) sc->flush_outbox();
}

int RdmaSendComm::post_stripes(RdmaSendReq* r) {
  RdmaEndpoint* e = rep();
  if (r->bounce_ev) {   // the device source is still on its way into the bounce buffer
    const int q = cuda::event_query(r->bounce_ev);
    if (q == 1) return -EINPROGRESS;
    if (q < 0) return -EIO;
    e->give_event(r->bounce_ev);
    r->bounce_ev = nullptr;
  }
  const MrTableEntry* mr = FabricEndpoint::mr_lookup(peer, r->target.mr_key);
  const uint32_t kind = r->via_frags ? static_cast<uint32_t>(MrKind::CUDA_STAGED)
                                     : (mr ? mr->kind : static_cast<uint32_t>(MrKind::HOST));
  const bool src_dev = r->bounce.empty() && r->src_dev;
  const char* src = r->bounce.empty() ? static_cast<const char*>(r->data) : reinterpret_cast<const char*>(r->bounce.data());
  bool all_done = true;
  bool back_pressure = false;   // some ring was full: the post must be retried in order
  for (int si = 0; si < r->nstripes; ++si) {
    Stripe& s = r->stripes[si];
    if (!s.complete && s.len == 0) {
      // NCCL posts empty messages (a ring step that carries no data still hands over a slot):
      // nothing to move, so no launch and no copy; only the completion travels
      s.posted = true;
      s.complete = true;
      B200NET_TRACE_EVENT(SendWriteSegmentStart, dev_id, local_comm_id, r->seq, s.len, r);
    }
    if (!s.complete) {
      if (kind == static_cast<uint32_t>(MrKind::CUDA_IPC) || kind == static_cast<uint32_t>(MrKind::CUDA_VMM)) {
        if (!s.posted) {
          void* mapped = e->map_peer_cuda(peer, mr);
          cuda::Stream st = e->rail_stream(s.rail);
          if (!mapped || !st) return -EIO;
          // the peer's address minus the base of the allocation its handle stands for, applied to
          // what the open of that handle returned here; never outside that allocation
          if (r->target.buff_addr < mr->base || r->target.buff_addr + r->size > mr->base + mr->size) {
            NET_WARN("receive buffer %#llx+%zu lies outside its registration %#llx+%llu", static_cast<unsigned long long>(r->target.buff_addr),
                     r->size, static_cast<unsigned long long>(mr->base), static_cast<unsigned long long>(mr->size));
            return -EINVAL;
          }
          char* dst = static_cast<char*>(mapped) + (r->target.buff_addr - mr->base) + s.offset;
          // The plugin's own copy kernel moves the stripe over NVLink and sets a completion word in
          // pinned memory: from a device source, or from a page-locked host source through the
          // address kernels read it at. The copy engine is the path of a run without the kernels
          // only: a copy-engine transfer into a peer's memory, queued while a collective kernel
          // runs on this device, was seen never to complete.
          const char* ksrc = src_dev ? src : (r->bounce.empty() ? r->src_alias : nullptr);
          NetKernels* nk = ksrc ? e->kernels : nullptr;
          const bool timing = PluginStats::get().histograms_on();
          const uint64_t t0 = timing ? PluginStats::now_ns() : 0;
          // on the shared stream a stripe may share its launch with the stripes posted around it
          const bool queued = nk && st == nk->stream() && params().copy_batch.get();
          if (nk && (queued ? nk->copy_queue(dst, ksrc + s.offset, s.len, &s.kslot, src_dev)
                            : nk->copy_flag(dst, ksrc + s.offset, s.len, st, 0, &s.kslot, src_dev)) == 0) {
            e->bytes_kernel += s.len;
            if (timing) {
              s.t_launch_ns = PluginStats::now_ns();
              PluginStats::get().sample_launch(s.t_launch_ns - t0);
            }
          } else {
            s.kslot = -1;
            s.event = e->take_event();
            if (!s.event || cuda::memcpy_async(dst, src + s.offset, s.len, st) != 0 || cuda::event_record(s.event, st) != 0) return -EIO;
            e->bytes_copy_engine += s.len;
          }
          s.posted = true;
          B200NET_TRACE_EVENT(SendWriteSegmentStart, dev_id, local_comm_id, r->seq, s.len, r);
        }
        if (s.kslot >= 0) {
          NetKernels* nk = e->kernels;
          if (!nk) return -EIO;
          const int ks = nk->status(s.kslot);
          if (ks < 0) {
            NET_WARN("stripe of %zu bytes not delivered: its copy kernel could not be launched or gave up on a wait", s.len);
            nk->release(s.kslot);
            s.kslot = -1;
            return ks;
          }
          if (ks == 1) {
            nk->release(s.kslot);
            s.kslot = -1;
            s.done = s.len;
            s.complete = true;
            if (s.t_launch_ns) PluginStats::get().sample_kernel_done(PluginStats::now_ns() - s.t_launch_ns);
          }
        } else {
          const int q = cuda::event_query(s.event);
          if (q < 0) return -EIO;
          if (q == 0) {
            e->give_event(s.event);
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
      WriteCompletion wc{remote_comm_id, r->seq, r->recv_idx, static_cast<uint8_t>(r->nstripes), s.len};
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
  if (mappable && !r->src_dev && r->size && rep()->kernels) {
    // host source, device destination: the copy kernel reads page-locked host memory in place;
    // pageable memory travels as fragments that the receiver copies into its own device
    void* alias = nullptr;
    if (cuda::host_device_alias(r->data, &alias) == 0) r->src_alias = static_cast<const char*>(alias);
    else r->via_frags = true;
  }
  if (mappable && !r->via_frags && !rep()->map_peer_cuda(peer, mr)) {
    // the peer's device memory cannot be mapped into this process (another container, a driver
    // without IPC) or its mapping has not arrived yet: the payload travels as fragments that the
    // receiver copies to its device
    rep()->note_unmapped(peer, mr);
    r->via_frags = true;
  }
  if ((dst_host || r->via_frags || (mr && mr->kind == static_cast<uint32_t>(MrKind::CUDA_STAGED))) && r->size && r->src_dev) {
    // device source, destination only reachable through host memory: fetch it once; the stripes
    // start when the event behind the copy has completed (post_stripes polls it)
    r->bounce.resize(r->size);
    cuda::Stream st = rep()->rail_stream(0);
    r->bounce_ev = rep()->take_event();
    if (!st || !r->bounce_ev || cuda::memcpy_async(r->bounce.data(), r->data, r->size, st) != 0 ||
        cuda::event_record(r->bounce_ev, st) != 0)
      return -EIO;
  }
  Schedule* sc = sched->get_schedule(r->size, rep()->num_rails);
  if (!sc) return -ENOMEM;
  r->nstripes = 0;
  for (size_t i = 0; i < sc->num_xfer_infos && i < static_cast<size_t>(MAX_NUM_RAILS); ++i) {
    Stripe& s = r->stripes[r->nstripes++];
    s = Stripe{};
    s.rail = sc->xfers[i].rail_id;
    s.offset = sc->xfers[i].offset;
    s.len = sc->xfers[i].msg_size;
  }
  sched->release_schedule(sc);
  r->state = ReqState::PENDING;
  return 0;
}

int RdmaSendComm::send(void* data, size_t size, int tag, MrHandle* mh, Request** req) {
  RdmaEndpoint* e = rep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *req = nullptr;
  if (!e->is_active()) return -ECONNABORTED;
  if (peer_closed) return -ENOTCONN;
  e->progress();
  if (!e->is_active()) return -ECONNABORTED;
  if (inflight >= NET_MAX_SEND_REQUESTS) return 0;
  bind_eager_queue();
  const bool src_is_device = size > 0 && (mh ? mh->type == NCCL_PTR_CUDA : !cuda::is_host_pointer(data));
  auto* box = static_cast<CtrlMsg*>(mailbox->data());
  int n = 0;
  // a send may take an entry directly unless an eager send of the same tag is still waiting for
  // one (it has to go first); then it queues behind that one (-3: eager if small, else refused)
  const int idx = tag_is_queued(tag) ? -3 : match_entry(box[next_seq % MAILBOX_SLOTS], next_seq, consumed_mask, tag, &n);
  NET_TRACE(NCCL_NET, "send: seq %u idx %d eagerq %zu ready0 %x size %zu", next_seq, idx, eager_queue.size(),
            box[next_seq % MAILBOX_SLOTS].entries[0].ready.load(), size);
  if (idx >= 0) {
    RdmaSendReq* r = e->send_reqs.take();
    if (!r) return 0;   // pool exhausted: NCCL calls again after completions
    r->comm = this;
    r->data = data;
    r->size = size;
    r->tag = tag;
    r->seq = next_seq;
    r->recv_idx = static_cast<uint8_t>(idx);
    r->src_dev = src_is_device;
    r->serial = e->next_req_serial++;
    ++inflight;
    e->live_send_reqs[r->serial] = r;
    const int rc = start_rendezvous(r, box[next_seq % MAILBOX_SLOTS].entries[idx]);
    if (rc != 0) {
      release(r);
      return rc;
    }
    B200NET_TRACE_EVENT(Send, dev_id, local_comm_id, r->seq, r->size, r);
    PluginStats::bump(PluginStats::get().rendezvous_sends);
    consume_entry(idx, n);
    bind_eager_queue();   // if that completed the group, queued sends may fit the next one
    const int prc = post_stripes(r);
    if (prc != 0 && prc != -EAGAIN && prc != -EINPROGRESS) {
      r->state = ReqState::ERROR;
    } else if (prc == -EAGAIN) {
      B200NET_TRACE_EVENT(PendingQueueInsert, dev_id, local_comm_id, r->seq, r->size, r);
      e->pending.push_back(r->serial);
    }
    e->note_activity();
    ++accepted;
    refused_since = 0;
    *req = r;
    return 0;
  }
  // no control message yet: eager if allowed
  const size_t eager_max = params().eager_max_size.get();
  const bool eager_size_ok = eager_max > 0 && size <= eager_max && size + sizeof(EagerHdr) <= FAB_LARGE_CELL &&
                             static_cast<int>(eager_queue.size()) < MAX_EAGER_PENDING;
  if (!eager_size_ok) {
    ++refused_since;
    return 0;  // neither control message nor eager: *req stays null and NCCL retries
  }
  RdmaSendReq* r = e->send_reqs.take();
  if (!r) return 0;
  r->comm = this;
  r->data = data;
  r->size = size;
  r->tag = tag;
  r->eager = true;
  r->state = ReqState::PENDING;
  memset(&r->ehdr, 0, sizeof(r->ehdr));
  r->ehdr.remote_comm_id = remote_comm_id;
  r->ehdr.eager_seq = next_eager_seq;
  r->ehdr.base_seq = next_seq;
  r->ehdr.base_mask = consumed_mask;
  r->ehdr.tag = tag;
  r->ehdr.size = size;
  const bool dev_src = src_is_device;
  if (dev_src) {
    // device payload: the pack kernel writes header + payload + flag into a pinned slot; without
    // the kernels the copy engine fetches the payload into a staging slot. Either way the datagram
    // leaves from the outbox once the payload has arrived; this call does not wait for it.
    NetKernels* nk = size <= NetKernels::EAGER_PAYLOAD_MAX ? e->kernels : nullptr;
    cuda::Stream st = e->rail_stream(0);
    bool ok = st != nullptr;
    if (ok && !(nk && nk->eager_pack(data, size, next_eager_seq, size, st, &r->pack_slot) == 0)) {
      r->pack_slot = -1;
      r->stage = e->staging().entry_alloc();
      r->stage_ev = r->stage ? e->take_event() : nullptr;
      ok = r->stage && r->stage_ev && cuda::memcpy_async(r->stage->ptr, data, size, st) == 0 && cuda::event_record(r->stage_ev, st) == 0;
    }
    if (!ok) {
      e->give_event(r->stage_ev);
      if (r->stage) e->staging().entry_free(r->stage);
      e->send_reqs.give(r);
      return -EIO;
    }
  } else if (outbox.empty()) {
    const int rc = e->fab.send(peer, DgramType::EAGER, 0, &r->ehdr, sizeof(r->ehdr), data, size);
    if (rc != 0) {
      e->send_reqs.give(r);
      return rc == -EAGAIN ? 0 : rc;  // ring full: NCCL calls again
    }
    r->dgram_sent = true;
    e->bytes_eager += size;
    PluginStats::bump(PluginStats::get().eager_sends);
  }
  r->serial = e->next_req_serial++;
  e->live_send_reqs[r->serial] = r;
  ++next_eager_seq;
  ++inflight;
  eager_queue.push_back(r);
  if (!r->dgram_sent) {
    r->t_outbox_ns = PluginStats::now_ns();
    outbox.push_back(r);
    ++e->outbox_total;
    flush_outbox();
  }
  // an eager send learns its message sequence number when a receive is matched: until then it is
  // known by its eager sequence number (ranges are keyed by the request, not by the number)
  B200NET_TRACE_EVENT(Send, dev_id, local_comm_id, r->ehdr.eager_seq, size, r);
  B200NET_TRACE_EVENT(SendEagerStart, dev_id, local_comm_id, r->ehdr.eager_seq, size, r);
  e->note_activity();
  ++accepted;
  refused_since = 0;
  *req = r;
  return 0;
}

int RdmaSendReq::test(int* done, int* sizes) {
  RdmaEndpoint* e = comm->rep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *done = 0;
  if (!e->is_active()) return -ECONNABORTED;
  e->progress();
  if (!e->is_active()) return -ECONNABORTED;
  if (eager) {
    if (!dgram_sent && state != ReqState::ERROR) comm->flush_outbox();
    if (state == ReqState::PENDING) comm->bind_eager_queue();
  } else if (state == ReqState::PENDING) {
    const int rc = comm->post_stripes(this);
    if (rc != 0 && rc != -EAGAIN && rc != -EINPROGRESS) state = ReqState::ERROR;
  }
  if (state == ReqState::ERROR) {
    PluginStats::bump(PluginStats::get().requests_failed);
    comm->release(this);
    return -EIO;
  }
  if (state == ReqState::COMPLETED && (!eager || dgram_sent)) {
    *done = 1;
    if (sizes) sizes[0] = static_cast<int>(size);
    B200NET_TRACE_EVENT(SendEnd, comm->dev_id, comm->local_comm_id, seq, size, this);
    if (PluginStats::get().histograms_on()) PluginStats::get().sample_send(size, static_cast<size_t>(nstripes), PluginStats::since(t_post_ns));
    e->note_activity();
    comm->release(this);
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
    e->outbox_total -= static_cast<int>(outbox.size());
    outbox.clear();
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
RdmaRecvComm::~RdmaRecvComm() {
  for (EagerRx& rx : eager_rx)
    if (rx.slot) rep()->staging().entry_free(rx.slot);
}

void RdmaRecvComm::release(RdmaRecvReq* r) { rep()->recv_reqs.give(r); }

void RdmaRecvComm::finish_sub(RdmaRecvReq* r, int idx) {
  if (r->subs[idx].done) return;
  r->subs[idx].done = true;
  eager_taken[r->seq % MAILBOX_SLOTS] |= static_cast<uint8_t>(1u << idx);
  if (++r->ndone == r->n) {
    if (r->state != ReqState::ERROR) r->state = ReqState::COMPLETED;
    MsgStatus st;
    msgbuff->complete(r->seq, &st);
    posted.remove(r);
    if (r->user_released) release(r);
  }
}

// The payload of one sub-receive could not be delivered: the request reports an error from test()
// instead of a size (its other sub-receives still retire the bookkeeping).
void RdmaRecvComm::fail_sub(RdmaRecvReq* r, int idx) {
  r->state = ReqState::ERROR;
  PluginStats::bump(PluginStats::get().requests_failed);
  finish_sub(r, idx);
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
  rx.slot = nullptr;
  if (h.size) {
    rx.slot = h.size <= STAGE_BYTES ? rep()->staging().entry_alloc() : nullptr;
    if (!rx.slot) {
      rep()->fail_endpoint("no staging slot for an eager payload", -ENOMEM);
      return;
    }
    memcpy(rx.slot->ptr, data, h.size);
  }
  // keep the list ordered by eager_seq (datagrams of one sender arrive in order; be safe anyway)
  size_t at = eager_rx.size();
  while (at > 0 && static_cast<int16_t>(h.eager_seq - eager_rx[at - 1].hdr.eager_seq) < 0) --at;
  eager_rx.insert(eager_rx.begin() + static_cast<std::ptrdiff_t>(at), rx);
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
//
// A payload for host memory is copied at once. A payload for device memory is queued on the
// receive stream from its (page-locked) staging slot and the sub-receive completes when the event
// behind the copy has; nothing here waits for the device.
void RdmaRecvComm::match_eager() {
  RdmaEndpoint* e = rep();
  int blocked_tags[MAX_EAGER_PENDING + 1];
  int nblocked = 0;
  size_t at = 0;
  while (at < eager_rx.size()) {
    EagerRx& rx = eager_rx[at];
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
      ++at;
      continue;
    }
    SubRecv& s = target->subs[target_idx];
    const size_t nbytes = std::min<size_t>(rx.hdr.size, s.cap);
    FreelistEntry* slot = rx.slot;
    eager_rx.erase(eager_rx.begin() + static_cast<std::ptrdiff_t>(at));   // `rx` is gone from here on
    eager_taken[target->seq % MAILBOX_SLOTS] |= static_cast<uint8_t>(1u << target_idx);
    s.received = nbytes;
    if (nbytes && s.mem_type == NCCL_PTR_CUDA) {
      Deferred d;
      d.kind = Deferred::EAGER_COPY;
      d.slot = slot;
      d.comm_id = local_comm_id;
      d.seq = target->seq;
      d.idx = static_cast<uint8_t>(target_idx);
      const int rc = e->stage_to_device(s.buf, slot, nbytes, &d);
      if (rc != 0) {
        NET_WARN("copy of an eager payload to the device failed (%d)", rc);
        e->staging().entry_free(slot);
        fail_sub(target, target_idx);
        continue;
      }
      e->deferred.push_back(d);
      continue;
    }
    if (nbytes) memcpy(s.buf, slot->ptr, nbytes);
    if (slot) e->staging().entry_free(slot);
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
  if (!e->is_active()) return -ECONNABORTED;
  if (inflight >= NET_MAX_REQUESTS) return 0;
  // the mailbox slot of this sequence number must not still describe a live group
  const uint16_t seq = next_seq;
  RdmaRecvReq* r = e->recv_reqs.take();
  if (!r) return 0;
  r->comm = this;
  r->seq = seq;
  r->n = n;
  // Early completion is safe only when every byte reaches the buffer without this process's help
  // (a write into mapped or attached memory): after an early "done" NCCL may never call the plugin
  // again for this transfer, and eager payloads are delivered by the receiver's progress loop.
  r->no_completion = optional && params().early_completion.get() && params().eager_max_size.get() == 0;
  MsgStatus st;
  if (msgbuff->insert(seq, r, MsgElemType::REQ, &st) != MsgResult::SUCCESS) {
    release(r);
    return 0;  // window full: try again after completions
  }
  eager_taken[seq % MAILBOX_SLOTS] = 0;
  auto* box = static_cast<CtrlMsg*>(mailbox->data());
  CtrlMsg& slot = box[seq % MAILBOX_SLOTS];
  B200NET_TRACE_EVENT(WriteCtrlStart, dev_id, local_comm_id, seq, n, r);
  for (int i = 0; i < n; ++i) {
    r->subs[i] = SubRecv{data[i], sizes[i], tags[i], mh ? mh[i] : nullptr, (mh && mh[i]) ? mh[i]->type : NCCL_PTR_HOST};
    if (mh && mh[i]) {
      const int rc = e->ensure_published(mh[i]);   // device registrations were published when they were made
      if (rc != 0) {
        msgbuff->complete(seq, &st);
        release(r);
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
  e->note_activity();
  *req = r;
  return 0;
}

int RdmaRecvReq::test(int* done, int* sizes) {
  RdmaEndpoint* e = comm->rep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *done = 0;
  if (!e->is_active()) return -ECONNABORTED;
  e->progress();
  if (!e->is_active()) return -ECONNABORTED;
  if (state == ReqState::ERROR && ndone == n) {
    // a payload could not be delivered (its copy to the device failed)
    --comm->inflight;
    comm->release(this);
    return -EIO;
  }
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
    e->note_activity();
    comm->release(this);
  } else if (no_completion && state != ReqState::ERROR) {
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
  RdmaEndpoint* e = ep;
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  e->progress();
  *done = 1;
  e->flush_reqs.give(this);
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
  *req = e->flush_reqs.take(e);
  return *req ? 0 : -ENOMEM;
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
    // copies queued for this communicator's receives complete into nothing: keep only their slots and events
    for (Deferred& d : e->deferred)
      if (d.kind == Deferred::EAGER_COPY && d.comm_id == local_comm_id) d.kind = Deferred::FRAG_COPY;
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
