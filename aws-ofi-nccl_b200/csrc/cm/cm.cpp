#include "b200net/cm.h"

#include <cerrno>
#include <cstring>

#include "b200net/log.h"
#include "b200net/tracepoint.h"

namespace b200net {

ConnectionManager::ConnectionManager(FabricEndpoint* ep) : ep_(ep) {}

size_t ConnectionManager::pending_requests() const {
  std::lock_guard<std::mutex> g(mu_);
  return connectors_.size();
}

std::unique_ptr<CmListener> ConnectionManager::listen() {
  std::lock_guard<std::mutex> g(mu_);
  const uint64_t id = listener_ids_.allocate();
  if (id == IdPool::ID_NONE) return nullptr;
  auto l = std::unique_ptr<CmListener>(new CmListener());
  l->cm_ = this;
  l->id_ = static_cast<uint32_t>(id);
  listeners_[l->id_] = l.get();
  return l;
}

CmListener::~CmListener() {
  std::lock_guard<std::mutex> g(cm_->mu_);
  cm_->listeners_.erase(id_);
  cm_->listener_ids_.free_id(id_);
}

std::unique_ptr<CmReceiver> CmListener::accept() {
  std::lock_guard<std::mutex> g(cm_->mu_);
  if (ready_.empty()) return nullptr;
  auto r = std::move(ready_.front());
  ready_.pop_front();
  B200NET_TRACE_EVENT(CmAccept, 0, id_, 0, 0, r.get());
  return r;
}

std::unique_ptr<CmSendConnector> ConnectionManager::connect(const std::string& listener_ep, uint32_t listener_id,
                                                            const void* payload, size_t len) {
  if (len > CM_MAX_PAYLOAD) return nullptr;
  std::lock_guard<std::mutex> g(mu_);
  const uint64_t id = connector_ids_.allocate();
  if (id == IdPool::ID_NONE) return nullptr;
  auto c = std::unique_ptr<CmSendConnector>(new CmSendConnector());
  c->cm_ = this;
  c->id_ = static_cast<uint32_t>(id);
  c->listener_ep_ = listener_ep;
  c->listener_id_ = listener_id;
  c->payload_.assign(static_cast<const uint8_t*>(payload), static_cast<const uint8_t*>(payload) + len);
  connectors_[c->id_] = c.get();
  return c;
}

CmSendConnector::~CmSendConnector() {
  std::lock_guard<std::mutex> g(cm_->mu_);
  cm_->connectors_.erase(id_);
  cm_->connector_ids_.free_id(id_);
}

static void fill_msg(CmConnMsg* m, CmMsgType type, uint32_t local_id, uint32_t remote_id, const std::string& my_ep,
                     const std::vector<uint8_t>& payload) {
  memset(m, 0, sizeof(*m));
  m->type = static_cast<uint32_t>(type);
  m->local_id = local_id;
  m->remote_id = remote_id;
  m->payload_len = static_cast<uint32_t>(payload.size());
  strncpy(m->conn_ep_name, my_ep.c_str(), sizeof(m->conn_ep_name) - 1);
  if (!payload.empty()) memcpy(m->payload, payload.data(), payload.size());
}

int CmSendConnector::test_ready() {
  if (!sent_) {
    PeerMapping* peer = cm_->ep_->av_insert(listener_ep_);
    if (!peer) return -EHOSTUNREACH;
    CmConnMsg m;
    fill_msg(&m, CmMsgType::CONN, id_, listener_id_, cm_->ep_->name(), payload_);
    const int rc = cm_->ep_->send(peer, DgramType::CM_CONN, 0, &m, sizeof(m));
    if (rc == -EAGAIN) return 0;
    if (rc != 0) return rc;
    sent_ = true;
    B200NET_TRACE_EVENT(CmConnect, 0, id_, 0, payload_.size(), this);
  }
  std::lock_guard<std::mutex> g(cm_->mu_);
  return have_resp_ ? 1 : 0;
}

void CmReceiver::set_conn_resp_msg_data(const void* data, size_t len) {
  resp_payload_.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + len);
}

int CmReceiver::test_ready() {
  if (sent_) return 1;
  if (resp_payload_.size() > CM_MAX_PAYLOAD) return -EMSGSIZE;
  PeerMapping* peer = cm_->ep_->av_insert(peer_name_);
  if (!peer) return -EHOSTUNREACH;
  CmConnMsg m;
  fill_msg(&m, CmMsgType::CONN_RESP, local_id_, peer_connector_id_, cm_->ep_->name(), resp_payload_);
  const int rc = cm_->ep_->send(peer, DgramType::CM_CONN_RESP, 0, &m, sizeof(m));
  if (rc == -EAGAIN) return 0;
  if (rc != 0) return rc;
  sent_ = true;  // the fabric delivers or reports: no separate send completion to wait for
  B200NET_TRACE_EVENT(CmConnResp, 0, local_id_, 0, resp_payload_.size(), this);
  return 1;
}

bool ConnectionManager::handle_dgram(const DgramHdr& hdr, const void* payload) {
  if (hdr.type != static_cast<uint16_t>(DgramType::CM_CONN) && hdr.type != static_cast<uint16_t>(DgramType::CM_CONN_RESP))
    return false;
  if (hdr.len < offsetof(CmConnMsg, payload)) {
    NET_WARN("truncated connection-manager message (%u bytes) dropped", hdr.len);
    return true;
  }
  const CmConnMsg* m = static_cast<const CmConnMsg*>(payload);
  if (m->payload_len > CM_MAX_PAYLOAD || offsetof(CmConnMsg, payload) + m->payload_len > hdr.len) {
    NET_WARN("malformed connection-manager message dropped");
    return true;
  }
  std::lock_guard<std::mutex> g(mu_);
  if (m->type == static_cast<uint32_t>(CmMsgType::CONN)) {
    auto it = listeners_.find(m->remote_id);
    if (it == listeners_.end()) {
      NET_INFO(NCCL_NET, "connection request for unknown listener %u ignored", m->remote_id);
      return true;
    }
    auto r = std::unique_ptr<CmReceiver>(new CmReceiver());
    r->cm_ = this;
    r->peer_name_.assign(m->conn_ep_name, strnlen(m->conn_ep_name, sizeof(m->conn_ep_name)));
    r->peer_connector_id_ = m->local_id;
    r->local_id_ = m->remote_id;
    r->conn_payload_.assign(m->payload, m->payload + m->payload_len);
    it->second->ready_.push_back(std::move(r));
  } else {
    auto it = connectors_.find(m->remote_id);
    if (it == connectors_.end()) return true;  // connector already gone (closed while connecting)
    it->second->resp_payload_.assign(m->payload, m->payload + m->payload_len);
    it->second->have_resp_ = true;
  }
  return true;
}

}  // namespace b200net
