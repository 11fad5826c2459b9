// Connection manager: turns the connectionless fabric into NCCL's listen / connect / accept.
// A listener is identified by (endpoint name, listener id) — that pair is what travels in the
// 128-byte handle. The connector sends a CONN message carrying its own endpoint name, an id for
// the reply and a transport-specific payload; the acceptor answers with CONN_RESP carrying its
// payload. Both sides are polled: nothing here blocks
// (reference: include/cm/nccl_ofi_cm.h:27-220, src/cm/*.cpp).
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "b200net/idpool.h"
#include "b200net/shm_fabric.h"

namespace b200net {

constexpr size_t CM_MAX_PAYLOAD = 160;

enum class CmMsgType : uint32_t { CONN = 1, CONN_RESP = 2 };

struct CmConnMsg {
  uint32_t type;
  uint32_t local_id;    // id of the sender of this message (connector id, or receiver id)
  uint32_t remote_id;   // id at the destination (listener id for CONN, connector id for CONN_RESP)
  uint32_t payload_len;
  char conn_ep_name[FAB_EP_NAME_LEN];  // where to send the reply
  uint8_t payload[CM_MAX_PAYLOAD];
};
static_assert(sizeof(CmConnMsg) <= FAB_SMALL_CELL, "CM messages travel in the small ring");

class ConnectionManager;

// Acceptor side of one incoming connection.
class CmReceiver {
 public:
  const std::vector<uint8_t>& conn_msg_data() const { return conn_payload_; }
  const std::string& peer_ep_name() const { return peer_name_; }
  void set_conn_resp_msg_data(const void* data, size_t len);
  // Sends the response (retrying on back-pressure). 1 = sent, 0 = try again, <0 = error.
  int test_ready();

 private:
  friend class ConnectionManager;
  friend class CmListener;
  ConnectionManager* cm_ = nullptr;
  std::string peer_name_;
  uint32_t peer_connector_id_ = 0;
  uint32_t local_id_ = 0;
  std::vector<uint8_t> conn_payload_, resp_payload_;
  bool sent_ = false;
};

class CmListener {
 public:
  ~CmListener();
  uint32_t id() const { return id_; }
  // Next fully received connection request, or null.
  std::unique_ptr<CmReceiver> accept();

 private:
  friend class ConnectionManager;
  ConnectionManager* cm_ = nullptr;
  uint32_t id_ = 0;
  std::deque<std::unique_ptr<CmReceiver>> ready_;
};

// Connector side.
class CmSendConnector {
 public:
  ~CmSendConnector();
  // Sends the request if not sent yet; 1 once the response has arrived, 0 otherwise, <0 on error.
  int test_ready();
  const std::vector<uint8_t>& conn_resp_data() const { return resp_payload_; }

 private:
  friend class ConnectionManager;
  ConnectionManager* cm_ = nullptr;
  uint32_t id_ = 0;
  std::string listener_ep_;
  uint32_t listener_id_ = 0;
  std::vector<uint8_t> payload_, resp_payload_;
  bool sent_ = false, have_resp_ = false;
};

class ConnectionManager {
 public:
  explicit ConnectionManager(FabricEndpoint* ep);
  std::unique_ptr<CmListener> listen();
  std::unique_ptr<CmSendConnector> connect(const std::string& listener_ep, uint32_t listener_id, const void* payload,
                                           size_t len);
  // Feed CM datagrams popped by the owner's progress loop. Returns true if the type was a CM type.
  bool handle_dgram(const DgramHdr& hdr, const void* payload);
  FabricEndpoint* ep() { return ep_; }
  size_t pending_requests() const;

 private:
  friend class CmListener;
  friend class CmSendConnector;
  friend class CmReceiver;
  FabricEndpoint* ep_;
  mutable std::mutex mu_;
  IdPool listener_ids_{4096}, connector_ids_{32768};
  std::map<uint32_t, CmListener*> listeners_;
  std::map<uint32_t, CmSendConnector*> connectors_;
};

}  // namespace b200net
