// Object model of the net plugin: plugin -> device -> domain -> endpoint -> {listen, send, recv}
// communicators -> requests, plus memory-registration handles. The transports (RDMA-style and
// tagged send/recv) derive from these classes; the validated C API and the versioned ABI tables
// only see this header (reference: include/nccl_ofi.h:128-838).
#pragma once
#include <atomic>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "b200net/idpool.h"
#include "b200net/mr_cache.h"
#include "nccl_abi.h"

namespace b200net {

constexpr int NET_MAX_RECVS = 8;               // receives grouped in one irecv
constexpr int NET_MAX_REQUESTS = 128;          // in-flight receive requests per communicator
constexpr int NET_MAX_SEND_REQUESTS = 128 * 8; // in-flight send requests per communicator
constexpr int NET_FLUSH_SIZE = 4;
constexpr int NET_CACHELINE = 64;
constexpr size_t NET_MAX_EP_ADDR = 56;
constexpr int NET_MAX_COMMS = 32768;

// Stages of a non-blocking connect/accept, kept in the handle so the call is re-entrant.
enum class CommStage : int { COMM_CREATE_START = 0, COMM_SEND_CONN, COMM_RECV_CONN, COMM_CONN_REQ_PENDING,
                             COMM_CONN_RESP_REQ_PENDING, COMM_CONNECTED };

class SendComm;
struct SaveCommState {
  SendComm* comm;
  CommStage stage;
};

// The 128-byte blob NCCL carries from the listener to the connector.
struct ConnHandle {
  char ep_name[NET_MAX_EP_ADDR];
  uint32_t comm_id;     // listener id inside the endpoint's connection manager
  uint32_t reserved;
  SaveCommState state;  // used by the connecting side only
};
static_assert(sizeof(ConnHandle) <= NCCL_NET_HANDLE_MAXSIZE, "connect handle must fit NCCL's handle blob");

// Transport-independent view of a device's properties (converted per ABI version by the shims).
struct Properties {
  std::string name;
  std::string pci_path;
  uint64_t guid = 0;
  int ptr_support = NCCL_PTR_HOST;
  int reg_is_global = 1;
  int force_flush = 0;
  int port_speed_mbps = 0;
  int port = 1;
  float latency_us = 0;
  int max_comms = NET_MAX_COMMS;
  int max_recvs = NET_MAX_RECVS;
  size_t max_p2p_bytes = 0;
  size_t max_coll_bytes = 0;
  int max_multi_request_size = 1;
  int16_t rail_id = -1, plane_id = -1;
  int num_rails = 1;
};

// How a peer reaches a registration: host memory; device memory with a legacy IPC handle; device
// memory without any mapping (payloads travel as fragments that the owner copies); device memory
// of the virtual-memory API, exported as a file descriptor that the peer duplicates and imports.
enum class MrKind : uint32_t { HOST = 1, CUDA_IPC = 2, CUDA_STAGED = 3, CUDA_VMM = 4 };

class Endpoint;
class Domain;
class Device;

struct MrHandle {
  uint64_t key = 0;      // published in the endpoint's MR table under this key
  void* base = nullptr;
  size_t size = 0;
  int type = NCCL_PTR_HOST;
  MrKind kind = MrKind::HOST;
  int refcnt = 1;
  Domain* domain = nullptr;
};

enum class ReqState : int { CREATED, PENDING, COMPLETED, ERROR };

class Request {
 public:
  virtual ~Request() = default;
  // Makes progress on the whole endpoint, then reports this request. sizes may be null.
  virtual int test(int* done, int* sizes) = 0;
  uint64_t t_post_ns = 0;   // when the post was accepted (steady clock); 0 unless latency histograms are on
};

class Comm {
 public:
  virtual ~Comm() = default;
  Endpoint* ep = nullptr;
  int dev_id = 0;
  uint32_t local_comm_id = 0, remote_comm_id = 0;
};

class SendComm : public Comm {
 public:
  virtual int send(void* data, size_t size, int tag, MrHandle* mh, Request** req) = 0;
  virtual int close() = 0;
};
class RecvComm : public Comm {
 public:
  virtual int recv(int n, void** data, size_t* sizes, int* tags, MrHandle** mh, Request** req,
                   bool optional_completion) = 0;
  virtual int flush(int n, void** data, int* sizes, MrHandle** mh, Request** req) = 0;
  virtual int close() = 0;
};
class ListenComm : public Comm {
 public:
  // *recv stays null until the connection is complete.
  virtual int accept(RecvComm** recv) = 0;
  virtual int close() = 0;
};

class Endpoint : public std::enable_shared_from_this<Endpoint> {
 public:
  explicit Endpoint(Domain* d) : domain(d) {}
  virtual ~Endpoint() = default;
  virtual int listen(ConnHandle* handle, ListenComm** lcomm) = 0;
  // Re-entrant: *scomm stays null until connected; progress is kept in handle->state.
  virtual int connect(ConnHandle* handle, SendComm** scomm, int traffic_class) = 0;
  virtual int reg_mr(void* data, size_t size, int type, MrHandle** mh) = 0;
  virtual int reg_mr_dmabuf(void* data, size_t size, int type, uint64_t offset, int fd, MrHandle** mh) = 0;
  virtual int dereg_mr(MrHandle* mh) = 0;
  // After invalidate() every call on the endpoint fails fast (a communicator was torn down with
  // requests in flight, so the endpoint's queues can no longer be trusted).
  void invalidate();   // every later call on this endpoint fails fast (counted in the statistics)
  bool is_active() const { return active.load(); }
  Domain* domain;
  std::shared_ptr<Domain> domain_ref;  // keeps the domain (MR cache, key pool, thread table) alive
  std::recursive_mutex ep_lock;
  std::atomic<bool> active{true};
};

class Domain : public std::enable_shared_from_this<Domain> {
 public:
  explicit Domain(Device* d);
  virtual ~Domain();
  virtual std::shared_ptr<Endpoint> create_endpoint() = 0;
  // One endpoint per calling thread (NCCL drives each proxy thread separately).
  std::shared_ptr<Endpoint> get_ep();
  Device* device;
  std::unique_ptr<MrCache> mr_cache;  // null when MR_CACHE_DISABLE
  IdPool mr_keys;
  std::mutex lock;

 private:
  std::map<long, std::weak_ptr<Endpoint>> ep_table_;  // keyed by thread id
};

class Device {
 public:
  Device(int id, std::string name) : dev_id(id), name(std::move(name)) {}
  virtual ~Device() = default;
  virtual int get_properties(Properties* props) = 0;
  virtual std::shared_ptr<Domain> create_domain() = 0;
  std::shared_ptr<Domain> get_domain();  // one domain per process per device
  std::shared_ptr<Endpoint> get_ep() { return get_domain()->get_ep(); }
  int dev_id;
  std::string name;
  int gpu_ordinal = -1;  // CUDA device this net device is closest to (-1: none / host only)

 private:
  std::mutex lock_;
  std::weak_ptr<Domain> domain_;
};

class Plugin {
 public:
  virtual ~Plugin() = default;
  int num_devices() const { return static_cast<int>(devices.size()); }
  Device* device(int i) { return i >= 0 && i < num_devices() ? devices[i].get() : nullptr; }
  std::vector<std::unique_ptr<Device>> devices;
  std::string protocol;  // "RDMA" or "SENDRECV"
};

// Plugin life cycle (net.cpp). create is idempotent under a reference count.
int net_create_plugin(Plugin** out);
Plugin* net_plugin();  // null before init
void net_destroy_plugin();

// Transport factories.
int rdma_create_devices(Plugin* p, int ndev, int num_rails);
int sendrecv_create_devices(Plugin* p, int ndev);

long current_tid();
// Name, PCI path, GUID, speed, latency and pointer support shared by both transports (net.cpp).
int fill_common_properties(Device* d, Properties* p, int rails);

}  // namespace b200net
