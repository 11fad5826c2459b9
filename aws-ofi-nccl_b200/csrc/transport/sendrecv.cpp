// Tagged send/receive transport: the simple protocol for fabrics without remote writes. Every
// message travels as fragments tagged with the communicator's id; the receiver matches them to
// posted receives in order, buffering fragments that arrive early. One receive per irecv, no
// grouped receives, registrations are per communicator
// (reference: src/nccl_ofi_sendrecv.cpp — send :1688-1775, recv :890-991, test :437-487,
//  properties :99-110).
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <deque>
#include <list>

#include "b200net/cm.h"
#include "b200net/cuda_shim.h"
#include "b200net/log.h"
#include "b200net/net.h"
#include "b200net/param.h"
#include "b200net/plugin_stats.h"
#include "b200net/shm_fabric.h"
#include "b200net/tracepoint.h"

namespace b200net::sendrecv {

struct FragHdr {
  uint32_t remote_comm_id;
  int32_t tag;
  uint32_t msg_seq;
  uint32_t pad;
  uint64_t offset, total;
};
struct ConnPayload { uint32_t comm_id; };

class SrEndpoint;
class SrSendComm;
class SrRecvComm;

class SrSendReq : public Request {
 public:
  int test(int* done, int* sizes) override;
  SrSendComm* comm;
  const char* data;
  size_t size, sent = 0;
  int tag;
  uint32_t msg_seq;
  bool staged = false;
  std::vector<uint8_t> bounce;
};
class SrRecvReq : public Request {
 public:
  int test(int* done, int* sizes) override;
  SrRecvComm* comm;
  char* buf;
  size_t cap, received = 0, total = ~size_t{0};
  int tag;
  uint32_t msg_seq;
  int mem_type = NCCL_PTR_HOST;  // copied at post time: the registration may be released before the data lands
  bool complete = false;
};
class SrFlushReq : public Request {
 public:
  int test(int* done, int*) override { *done = 1; delete this; return 0; }
};

struct EarlyFrag { FragHdr h; std::vector<uint8_t> data; };

class SrEndpoint : public Endpoint {
 public:
  explicit SrEndpoint(Domain* d) : Endpoint(d), cm(&fab) {}
  int listen(ConnHandle* handle, ListenComm** lcomm) override;
  int connect(ConnHandle* handle, SendComm** scomm, int) override;
  int reg_mr(void* data, size_t size, int type, MrHandle** mh) override {
    auto* h = new MrHandle();
    h->base = data; h->size = size; h->type = type; h->domain = domain;
    h->kind = type == NCCL_PTR_CUDA ? MrKind::CUDA_STAGED : MrKind::HOST;
    *mh = h;
    return 0;
  }
  int reg_mr_dmabuf(void* data, size_t size, int type, uint64_t, int, MrHandle** mh) override { return reg_mr(data, size, type, mh); }
  int dereg_mr(MrHandle* mh) override { delete mh; return 0; }
  void progress();
  FabricEndpoint fab;
  ConnectionManager cm;
  IdPool comm_ids{NET_MAX_COMMS};
  std::map<uint32_t, SrRecvComm*> recv_comms;
  std::map<uint32_t, SrSendComm*> send_comms;
  bool in_progress = false;
};

class SrSendComm : public SendComm {
 public:
  int send(void* data, size_t size, int tag, MrHandle* mh, Request** req) override;
  int close() override;
  int push(SrSendReq* r);
  int drive();
  SrEndpoint* sep() { return static_cast<SrEndpoint*>(ep); }
  std::unique_ptr<CmSendConnector> connector;
  PeerMapping* peer = nullptr;
  uint32_t next_msg = 0;
  std::deque<SrSendReq*> queue;  // messages go out strictly in order
  int inflight = 0;
  int failed = 0;
};

class SrRecvComm : public RecvComm {
 public:
  int recv(int n, void** data, size_t* sizes, int* tags, MrHandle** mh, Request** req, bool) override;
  int flush(int, void**, int*, MrHandle**, Request** req) override { *req = new SrFlushReq(); return 0; }
  int close() override;
  void on_frag(const FragHdr& h, const void* data, size_t len);
  void apply(SrRecvReq* r, const FragHdr& h, const void* data, size_t len);
  SrEndpoint* sep() { return static_cast<SrEndpoint*>(ep); }
  uint32_t next_msg = 0;
  std::deque<SrRecvReq*> posted;
  std::list<EarlyFrag> early;
  int inflight = 0;
};

class SrListenComm : public ListenComm {
 public:
  int accept(RecvComm** out) override;
  int close() override { listener.reset(); delete this; return 0; }
  std::unique_ptr<CmListener> listener;
  std::unique_ptr<CmReceiver> receiver;
  SrRecvComm* pending = nullptr;
};

void SrEndpoint::progress() {
  if (in_progress) return;
  in_progress = true;
  const int got = fab.poll(params().cq_read_count.get() * 16, [this](const DgramHdr& h, const void* p) {
    if (cm.handle_dgram(h, p)) return;
    if (h.type == static_cast<uint16_t>(DgramType::SENDRECV_FRAG) && h.len >= sizeof(FragHdr)) {
      const auto* fh = static_cast<const FragHdr*>(p);
      auto it = recv_comms.find(fh->remote_comm_id);
      if (it != recv_comms.end())
        it->second->on_frag(*fh, static_cast<const char*>(p) + sizeof(FragHdr), h.len - sizeof(FragHdr));
      else
        NET_WARN("fragment for unknown communicator %u dropped", fh->remote_comm_id);
    }
  });
  if (got > 0)
    B200NET_TRACE_EVENT(ProcessCompletionsSendRecv, domain->device->dev_id, 0, 0, static_cast<uint64_t>(got), this);
  // any call that makes progress also pushes queued sends of every communicator
  for (auto& [id, sc] : send_comms) sc->drive();
  in_progress = false;
}

int SrEndpoint::listen(ConnHandle* handle, ListenComm** lcomm) {
  std::lock_guard<std::recursive_mutex> g(ep_lock);
  auto l = std::make_unique<SrListenComm>();
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

int SrEndpoint::connect(ConnHandle* handle, SendComm** scomm, int) {
  std::lock_guard<std::recursive_mutex> g(ep_lock);
  *scomm = nullptr;
  auto* sc = static_cast<SrSendComm*>(handle->state.comm);
  if (!sc) {
    const uint64_t id = comm_ids.allocate();
    if (id == IdPool::ID_NONE) return -ENOSPC;
    sc = new SrSendComm();
    sc->ep = this;
    sc->dev_id = domain->device->dev_id;
    sc->local_comm_id = static_cast<uint32_t>(id);
    const std::string peer_name(handle->ep_name, strnlen(handle->ep_name, sizeof(handle->ep_name)));
    ConnPayload p{sc->local_comm_id};
    sc->connector = cm.connect(peer_name, handle->comm_id, &p, sizeof(p));
    sc->peer = fab.av_insert(peer_name);
    if (!sc->connector || !sc->peer) {
      comm_ids.free_id(id);
      delete sc;
      return -EHOSTUNREACH;
    }
    handle->state.comm = sc;
    handle->state.stage = CommStage::COMM_SEND_CONN;
  }
  progress();
  const int rc = sc->connector->test_ready();
  if (rc < 0) return rc;
  if (rc == 0) return 0;
  const auto& resp = sc->connector->conn_resp_data();
  if (resp.size() < sizeof(ConnPayload)) return -EPROTO;
  sc->remote_comm_id = reinterpret_cast<const ConnPayload*>(resp.data())->comm_id;
  sc->connector.reset();
  send_comms[sc->local_comm_id] = sc;
  handle->state.comm = nullptr;
  handle->state.stage = CommStage::COMM_CONNECTED;
  *scomm = sc;
  return 0;
}

int SrListenComm::accept(RecvComm** out) {
  auto* e = static_cast<SrEndpoint*>(ep);
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *out = nullptr;
  e->progress();
  if (!receiver) {
    receiver = listener->accept();
    if (!receiver) return 0;
    if (receiver->conn_msg_data().size() < sizeof(ConnPayload)) return -EPROTO;
    const uint64_t id = e->comm_ids.allocate();
    if (id == IdPool::ID_NONE) return -ENOSPC;
    pending = new SrRecvComm();
    pending->ep = e;
    pending->dev_id = dev_id;
    pending->local_comm_id = static_cast<uint32_t>(id);
    pending->remote_comm_id = reinterpret_cast<const ConnPayload*>(receiver->conn_msg_data().data())->comm_id;
    e->recv_comms[pending->local_comm_id] = pending;
    ConnPayload resp{pending->local_comm_id};
    receiver->set_conn_resp_msg_data(&resp, sizeof(resp));
  }
  const int rc = receiver->test_ready();
  if (rc < 0) return rc;
  if (rc == 0) return 0;
  *out = pending;
  pending = nullptr;
  receiver.reset();
  return 0;
}

// Push as many fragments of the head message as the peer's ring takes.
int SrSendComm::push(SrSendReq* r) {
  const size_t chunk = FAB_LARGE_CELL - sizeof(FragHdr) - 64;
  do {
    const size_t n = std::min(chunk, r->size - r->sent);
    FragHdr h{remote_comm_id, r->tag, r->msg_seq, 0, r->sent, r->size};
    const int rc = sep()->fab.send(peer, DgramType::SENDRECV_FRAG, 0, &h, sizeof(h), r->data + r->sent, n);
    if (rc != 0) return rc;
    r->sent += n;
  } while (r->sent < r->size);
  return 0;
}

// Push queued messages, strictly in order, until the peer's ring is full.
int SrSendComm::drive() {
  while (!queue.empty()) {
    SrSendReq* head = queue.front();
    const int rc = push(head);
    if (rc == -EAGAIN) return 0;
    if (rc != 0) {
      failed = rc;
      return rc;
    }
    head->staged = true;
    queue.pop_front();
  }
  return 0;
}

int SrSendComm::send(void* data, size_t size, int tag, MrHandle*, Request** req) {
  SrEndpoint* e = sep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *req = nullptr;
  if (!e->is_active()) return -ECONNABORTED;
  e->progress();
  if (inflight >= NET_MAX_REQUESTS) return 0;
  auto* r = new SrSendReq();
  r->comm = this;
  r->size = size;
  r->tag = tag;
  r->msg_seq = next_msg++;
  if (size && !cuda::is_host_pointer(data)) {  // device source: one bounce through host memory
    r->bounce.resize(size);
    cuda::Stream st = nullptr;
    if (cuda::stream_create(&st) != 0 || cuda::memcpy_async(r->bounce.data(), data, size, st) != 0 ||
        cuda::stream_synchronize(st) != 0) {
      delete r;
      return -EIO;
    }
    cuda::stream_destroy(st);
    r->data = reinterpret_cast<const char*>(r->bounce.data());
  } else {
    r->data = static_cast<const char*>(data);
  }
  queue.push_back(r);
  ++inflight;
  B200NET_TRACE_EVENT(Send, dev_id, local_comm_id, r->msg_seq, size, r);
  *req = r;
  return 0;
}

int SrSendReq::test(int* done, int* sizes) {
  SrEndpoint* e = comm->sep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *done = 0;
  if (!e->is_active()) return -ECONNABORTED;
  e->progress();
  if (comm->failed) return comm->failed;
  if (staged) {
    *done = 1;
    if (sizes) sizes[0] = static_cast<int>(size);
    B200NET_TRACE_EVENT(SendEnd, comm->dev_id, comm->local_comm_id, msg_seq, size, this);
    if (PluginStats::get().histograms_on()) PluginStats::get().sample_send(size, 1, PluginStats::since(t_post_ns));
    --comm->inflight;
    delete this;
  }
  return 0;
}

int SrSendComm::close() {
  SrEndpoint* e = sep();
  {
    std::lock_guard<std::recursive_mutex> g(e->ep_lock);
    if (inflight > 0) e->invalidate();
    e->send_comms.erase(local_comm_id);
    e->comm_ids.free_id(local_comm_id);
  }
  delete this;
  return 0;
}

void SrRecvComm::apply(SrRecvReq* r, const FragHdr& h, const void* data, size_t len) {
  r->total = h.total;
  if (h.offset < r->cap) {
    const size_t n = std::min(len, r->cap - static_cast<size_t>(h.offset));
    if (r->mem_type == NCCL_PTR_CUDA) {
      cuda::Stream st = nullptr;
      if (cuda::stream_create(&st) == 0) {
        cuda::memcpy_async(r->buf + h.offset, data, n, st);
        cuda::stream_synchronize(st);
        cuda::stream_destroy(st);
      }
    } else {
      if (n) memcpy(r->buf + h.offset, data, n);
    }
  }
  r->received += len;
  if (r->received >= r->total) r->complete = true;
}

void SrRecvComm::on_frag(const FragHdr& h, const void* data, size_t len) {
  for (SrRecvReq* r : posted) {
    if (r->msg_seq == h.msg_seq) {
      apply(r, h, data, len);
      return;
    }
  }
  EarlyFrag ef;
  ef.h = h;
  ef.data.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + len);
  early.push_back(std::move(ef));
}

int SrRecvComm::recv(int n, void** data, size_t* sizes, int* tags, MrHandle** mh, Request** req, bool) {
  SrEndpoint* e = sep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *req = nullptr;
  if (!e->is_active()) return -ECONNABORTED;
  if (n != 1) return -EINVAL;  // this protocol does not group receives
  e->progress();
  if (inflight >= NET_MAX_REQUESTS) return 0;
  auto* r = new SrRecvReq();
  r->comm = this;
  r->buf = static_cast<char*>(data[0]);
  r->cap = sizes[0];
  r->tag = tags[0];
  r->mem_type = (mh && mh[0]) ? mh[0]->type : NCCL_PTR_HOST;
  r->msg_seq = next_msg++;
  posted.push_back(r);
  ++inflight;
  for (auto it = early.begin(); it != early.end();) {
    if (it->h.msg_seq == r->msg_seq) {
      apply(r, it->h, it->data.data(), it->data.size());
      it = early.erase(it);
    } else {
      ++it;
    }
  }
  B200NET_TRACE_EVENT(Recv, dev_id, local_comm_id, r->msg_seq, 1, r);
  *req = r;
  return 0;
}

int SrRecvReq::test(int* done, int* sizes) {
  SrEndpoint* e = comm->sep();
  std::lock_guard<std::recursive_mutex> g(e->ep_lock);
  *done = 0;
  if (!e->is_active()) return -ECONNABORTED;
  e->progress();
  if (complete || total == 0) {
    *done = 1;
    if (sizes) sizes[0] = static_cast<int>(std::min(received, cap));
    for (auto it = comm->posted.begin(); it != comm->posted.end(); ++it)
      if (*it == this) {
        comm->posted.erase(it);
        break;
      }
    B200NET_TRACE_EVENT(RecvEnd, comm->dev_id, comm->local_comm_id, msg_seq, 1, this);
    PluginStats::bump(PluginStats::get().recv_bytes, std::min(received, cap));
    if (PluginStats::get().histograms_on()) PluginStats::get().sample_recv(std::min(received, cap), PluginStats::since(t_post_ns));
    --comm->inflight;
    delete this;
  }
  return 0;
}

int SrRecvComm::close() {
  SrEndpoint* e = sep();
  {
    std::lock_guard<std::recursive_mutex> g(e->ep_lock);
    if (inflight > 0) e->invalidate();
    e->recv_comms.erase(local_comm_id);
    e->comm_ids.free_id(local_comm_id);
  }
  delete this;
  return 0;
}

class SrDomain : public Domain {
 public:
  using Domain::Domain;
  std::shared_ptr<Endpoint> create_endpoint() override { return std::make_shared<SrEndpoint>(this); }
};
class SrDevice : public Device {
 public:
  SrDevice(int id, std::string n, int gpu) : Device(id, std::move(n)) { gpu_ordinal = gpu; }
  std::shared_ptr<Domain> create_domain() override { return std::make_shared<SrDomain>(this); }
  int get_properties(Properties* p) override {
    const int rc = fill_common_properties(this, p, 1);
    if (rc) return rc;
    p->max_recvs = 1;
    p->reg_is_global = 0;
    p->max_p2p_bytes = static_cast<size_t>(INT32_MAX);
    p->max_coll_bytes = static_cast<size_t>(INT32_MAX);
    return 0;
  }
};

}  // namespace b200net::sendrecv

namespace b200net {
int sendrecv_create_devices(Plugin* p, int ndev) {
  const int ngpu = cuda::device_count();
  for (int i = 0; i < ndev; ++i) {
    char name[64];
    snprintf(name, sizeof(name), "nvl%d", i);
    p->devices.push_back(std::make_unique<sendrecv::SrDevice>(i, name, i < ngpu ? i : -1));
  }
  p->protocol = "SENDRECV";
  return 0;
}
}  // namespace b200net
