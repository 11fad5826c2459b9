// GIN / RMA host side: collective connect, symmetric memory registration, put / put+signal / get /
// flush driven from the host ("proxy mode"), plus context creation for the kernel-initiated mode,
// where the plugin only lays out a GPU-resident handle block and the kernels do the rest
// (reference: src/rdma/gin/nccl_ofi_gin.cpp, nccl_ofi_gin_api.cpp, nccl_ofi_gin_gdaki.cpp,
//  include/rdma/gin/nccl_ofi_gin_types.h).
#pragma once
#include <atomic>
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "b200net/cuda_shim.h"
#include "b200net/mpsc_ring.h"
#include "b200net/net.h"
#include "b200net/shm_fabric.h"
#include "b200net/spsc_ring.h"

namespace b200net::gin {

constexpr int GIN_MAX_COMMS = 1024;
constexpr uint32_t GIN_ACK_REQ_THRESHOLD = 4096;  // un-acknowledged operations allowed per peer
constexpr int GIN_MAX_BACKEND_VERSION = 1;
constexpr int GIN_MAX_CONTEXTS = 8192 / 32;
constexpr int GIN_MAX_SIGNALS_PER_CONTEXT = 4096;

// ---- wire ------------------------------------------------------------------------------------
struct PeerRecord {           // all-gathered at connect
  char ep_name[FAB_EP_NAME_LEN];
  uint32_t pid;
  uint32_t comm_id;
};
struct RemoteMr {             // all-gathered at registration
  uint64_t addr, size, key;
  uint32_t kind, device;
  uint8_t ipc_handle[64];
};
struct MetadataMsg {          // "the put with this sequence number carries a signal"
  uint32_t comm_id;
  uint32_t src_rank;
  uint64_t seq;
  uint64_t signal_addr;       // absolute address at the target
  uint64_t signal_value;
  uint32_t signal_op;         // NCCL_NET_SIGNAL_OP_INC / ADD
  uint32_t signal_is_device;
};
struct AckMsg {
  uint32_t comm_id;
  uint32_t src_rank;
  uint64_t acked_seq;         // every operation up to and including this one has been applied
};

struct ReadReqMsg {           // "write [addr, addr+len) of your memory to my address reply_addr"
  uint32_t comm_id;
  uint32_t src_rank;
  uint64_t req_id;
  uint64_t addr, len, reply_addr;
};
struct ReadRespMsg {
  uint32_t comm_id;
  uint32_t src_rank;
  uint64_t req_id;
  int32_t status;
  uint32_t pad;
};

class CollComm;

struct SymmMr {
  void* base = nullptr;
  size_t size = 0;
  int type = NCCL_PTR_HOST;
  uint64_t flags = 0;
  MrHandle* local = nullptr;
  std::vector<RemoteMr> remote;     // indexed by rank
  std::vector<void*> mapped;        // device registrations: peer bases mapped into this process
  std::vector<size_t> mapped_bytes; // per peer: size of a virtual-memory-API mapping (0: legacy IPC)
  int export_fd = -1;               // descriptor kept open for peers that import this registration
  void* gpu_handle_block = nullptr; // kernel-initiated mode: peer base pointers in GPU memory
  int refcnt = 1;
};

class GinRequest {
 public:
  virtual ~GinRequest() = default;
  virtual int test(int* done) = 0;
};

struct PendingOp {            // a put whose data copy may still be running
  uint64_t seq = 0;
  cuda::Event event = nullptr;   // copy-engine transfer in flight (runs without the copy kernels)
  int kslot = -1;                // copy-kernel transfer in flight: its completion slot
  size_t len = 0, done = 0;
  uint64_t remote_addr = 0;
  const void* local = nullptr;
  std::vector<uint8_t> bounce;   // host copy of a device source that travels through host memory
  bool dev_frags = false;        // the target is device memory that cannot be mapped here: the owner
                                 // copies fragments to its device as they arrive
  bool has_signal = false, data_done = false, signal_sent = false, staged = false;
  MetadataMsg meta{};
  std::shared_ptr<std::atomic<int>> status;  // 0 pending, 1 done, <0 error (shared with the request)
};

struct PeerState {
  PeerMapping* map = nullptr;
  uint32_t comm_id = 0;
  uint64_t tx_head = 0;       // operations issued to this peer
  uint64_t tx_acked = 0;      // acknowledged by the peer
  uint64_t rx_applied = 0;    // operations from this peer applied here
  uint64_t rx_acked = 0;      // last acknowledgement sent to this peer
  std::deque<PendingOp> ops;  // retire strictly in order
};

// Work for the device-signal worker thread.
struct SignalWork {
  uint64_t addr;
  uint64_t value;   // amount to add
  uint32_t src_rank;
  uint32_t pad;
};

// One process-wide thread applies signal updates that target GPU memory: it keeps a host shadow of
// every signal word it has touched, folds updates to the same word, and writes the new value with
// an 8-byte copy, so the proxy thread never blocks on the GPU.
class DeviceSignalWorker {
 public:
  static DeviceSignalWorker& instance();
  bool submit(const SignalWork& w);   // false when the ring is full (caller retries)
  uint64_t completed() const { return completed_.load(); }
  uint64_t submitted() const { return submitted_.load(); }
  void drain();                       // wait until everything submitted so far is applied
  ~DeviceSignalWorker();

 private:
  DeviceSignalWorker();
  void run();
  MpscRing<SignalWork> ring_{4096};
  std::thread thread_;
  std::atomic<bool> stop_{false};
  std::atomic<uint64_t> submitted_{0}, completed_{0};
  std::map<uint64_t, uint64_t> shadow_;
  cuda::Stream stream_ = nullptr;
  // the context of the first caller that submitted work: the worker issues its copies in it (the
  // reference's worker likewise runs in the context captured when the communicator was made,
  // src/rdma/gin/nccl_ofi_gin.cpp:39-104)
  std::atomic<void*> ctx_{nullptr};
};

struct GinContext {
  CollComm* comm = nullptr;
  int n_signals = 0, n_counters = 0, n_contexts = 1;
  bool kernel_initiated = false;
  void* dev_pad = nullptr;            // kernel-initiated mode: this rank's signal/counter pad (GPU)
  std::vector<void*> peer_pads;       // peers' pads mapped here
  void* dev_handle_gpu = nullptr;     // GPU copy of the handle block
  ncclNetDeviceHandle_t net_dev_handle{};
  bool has_error = false;
};

class ListenComm {
 public:
  void* net_listen = nullptr;  // listen communicator of the net transport
  int dev = 0;
};

class CollComm {
 public:
  CollComm(int dev, int nranks, int rank);
  ~CollComm();
  // Ring connect (next / previous rank) over the net transport, then all-gather of the endpoint
  // records. Blocking with a deadline; collective.
  int connect(void* handles[], ListenComm* lcomm);
  // Ring all-gather of `bytes` per rank over the net transport's own send / recv (collective).
  int all_gather(void* buf, size_t bytes_per_rank);
  int reg_mr_sym(void* data, size_t size, int type, uint64_t flags, SymmMr** out);
  int dereg_mr_sym(SymmMr* mr);
  int create_context(int n_signals, int n_counters, int n_contexts, bool kernel_initiated, GinContext** out);
  int destroy_context(GinContext* ctx);
  int iput(uint64_t src_off, SymmMr* src, size_t size, uint64_t dst_off, SymmMr* dst, uint32_t rank, bool with_signal,
           uint64_t sig_off, SymmMr* sig, uint64_t sig_value, uint32_t sig_op, GinRequest** req);
  int iget(uint64_t remote_off, SymmMr* remote, size_t size, uint64_t local_off, SymmMr* local, uint32_t rank,
           GinRequest** req);
  int iflush(GinRequest** req);
  int progress();
  // Two-phase quiesce: stop issuing, wait until every peer has acknowledged everything, barrier.
  int close();
  bool has_error() const { return error_; }

  int dev, nranks, rank;
  uint32_t comm_id = 0;
  std::recursive_mutex lock;

 private:
  friend struct GinContext;
  void handle_dgram(const DgramHdr& h, const void* payload);
  int retire(PeerState& p, uint32_t peer_rank);
  int apply_signal(const MetadataMsg& m);
  int send_ack(uint32_t peer_rank);
  FabricEndpoint fab_;
  std::vector<PeerState> peers_;
  void* ring_send_ = nullptr;   // net send comm to rank+1
  void* ring_recv_ = nullptr;   // net recv comm from rank-1
  std::vector<SymmMr*> mrs_;
  std::vector<GinContext*> contexts_;
  std::deque<MetadataMsg> deferred_signals_;  // device signals the worker ring had no room for
  struct ReadService { ReadReqMsg req; size_t done; bool data_done; std::vector<uint8_t> bounce; };
  std::deque<ReadService> read_services_;     // reads this rank is serving for peers without direct access
  std::map<uint64_t, std::shared_ptr<std::atomic<int>>> reads_in_flight_;
  // a read served by the peer for a device destination lands in host memory first
  struct ReadLanding {
    std::vector<uint8_t> host;
    void* device_dst;
  };
  std::map<uint64_t, ReadLanding> read_landings_;
  uint64_t next_read_id_ = 1;
  int serve_reads();
  bool error_ = false, closing_ = false;
};

}  // namespace b200net::gin
