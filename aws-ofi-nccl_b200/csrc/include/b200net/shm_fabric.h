// The host-side "fabric" of one box: connectionless reliable endpoints built on POSIX shared
// memory. An endpoint owns a segment with two multi-producer rings (small cells for control,
// completions and connection-manager messages; large cells for eager payloads and staged write
// fragments); peers address it by name, map it once (the address vector) and push datagrams into
// its rings. Remote writes into registered host memory use cross-memory attach when the kernel
// allows it and fall back to fragments that the target applies in its progress loop.
//
// It stands where libfabric's FI_EP_RDM endpoints, address vector and completion queue stand in
// the reference (src/nccl_ofi_ofiutils.cpp, the CQ loop in src/nccl_ofi_rdma.cpp:1485-1568): same
// shape — post, -EAGAIN on back-pressure, poll for completions — different wire.
#pragma once
#include <sys/types.h>

#include <cstdint>
#include <condition_variable>
#include <deque>
#include <thread>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "b200net/mpsc_ring.h"

namespace b200net {

constexpr size_t FAB_EP_NAME_LEN = 56;       // fits the 56-byte address field of a connect handle
constexpr size_t FAB_SMALL_CELL = 240;       // bytes of payload per small-ring cell
constexpr size_t FAB_SMALL_CELLS = 4096;
constexpr size_t FAB_LARGE_CELL = 8192 + 64; // eager payload (8 KiB) + headers
constexpr size_t FAB_LARGE_CELLS = 256;
constexpr size_t FAB_MR_TABLE_SLOTS = 4096;

enum class DgramType : uint16_t {
  CM_CONN = 1, CM_CONN_RESP = 2, EAGER = 3, WRITE_COMPLETION = 4, WRITE_FRAG = 5, CLOSE = 6,
  GIN_METADATA = 7, GIN_ACK = 8, SENDRECV_MSG = 9, SENDRECV_FRAG = 10, READ_REQ = 11, READ_RESP = 12,
  USER = 100,
};

// send() flag: queue behind the large-cell traffic even if the datagram is small, so that it is
// seen only after fragments posted earlier (the two rings are not ordered against each other).
constexpr uint16_t DGRAM_FLAG_ORDER_AFTER_FRAGS = 0x1;

// First bytes of every datagram.
struct DgramHdr {
  uint16_t type;
  uint16_t flags;
  uint32_t src_ep_id;   // sender's endpoint id (index in its process)
  uint32_t src_pid;
  uint32_t len;         // payload bytes after the header
};

// What a peer needs to write into a registration (published in the owner's MR table).
struct MrTableEntry {
  uint64_t key;          // 0 = free
  uint64_t base;
  uint64_t size;
  uint32_t kind;         // 1 host, 2 cuda (ipc handle valid), 3 cuda staged (no direct mapping)
  uint32_t device;
  uint8_t ipc_handle[64];
  uint64_t serial;       // unique per publication in the owner's process (keys are recycled)
  uint8_t pad[24];
};
static_assert(sizeof(MrTableEntry) == 128, "MR table entries are 128 bytes");

struct EpSegmentHdr {
  uint64_t magic;
  uint32_t pid;
  uint32_t ep_id;
  uint64_t small_off, large_off, mr_table_off, total_bytes;
  std::atomic<uint32_t> closed;
};

class FabricEndpoint;

// A mapped remote (or local) endpoint: the address-vector entry.
struct PeerMapping {
  std::string name;
  void* base = nullptr;
  size_t bytes = 0;
  uint32_t pid = 0;
  MpscByteRing small, large;
  MrTableEntry* mr_table = nullptr;
  EpSegmentHdr* hdr = nullptr;
  bool cma_ok = false;     // process_vm_writev to this pid works
  bool cma_probed = false;
};

using DgramHandler = std::function<void(const DgramHdr& hdr, const void* payload)>;

class FabricEndpoint {
 public:
  // Creates the shared segment "/b200net.<pid>.<id>"; throws std::runtime_error on failure.
  FabricEndpoint();
  ~FabricEndpoint();
  FabricEndpoint(const FabricEndpoint&) = delete;
  FabricEndpoint& operator=(const FabricEndpoint&) = delete;

  const std::string& name() const { return name_; }
  uint32_t id() const { return id_; }

  // Address vector: map the endpoint called `name` (cached). nullptr if it does not exist.
  PeerMapping* av_insert(const std::string& name);
  void av_remove(const std::string& name);

  // Post a datagram (header is filled in here). 0, -EAGAIN (ring full), -EMSGSIZE, -ENOTCONN (peer closed).
  int send(PeerMapping* dst, DgramType type, uint16_t flags, const void* a, size_t alen, const void* b = nullptr,
           size_t blen = 0);
  // Remote write into peer host memory: cross-memory attach, else WRITE_FRAG datagrams applied by
  // the target's progress loop. *done is the number of bytes already written and is advanced;
  // returns 0 when *done == len, -EAGAIN when the target's ring filled up (call again later),
  // -ENOTCONN / -EFAULT on failure.
  int write_host(PeerMapping* dst, uint64_t remote_addr, const void* local, size_t len, size_t* done);
  // Remote read from peer host memory (cross-memory attach only). -ENOTSUP without it.
  int read_host(PeerMapping* dst, uint64_t remote_addr, void* local, size_t len);

  // Drain up to `budget` datagrams from the own rings. WRITE_FRAG datagrams are applied here and
  // not shown to the handler. Returns the number processed.
  int poll(int budget, const DgramHandler& handler);

  // MR table (read by peers).
  int mr_publish(const MrTableEntry& e);   // 0 or -ENOSPC
  void mr_unpublish(uint64_t key);
  static const MrTableEntry* mr_lookup(const PeerMapping* peer, uint64_t key);

  // True when write_host() towards this peer goes through fragments rather than direct writes.
  bool writes_are_staged(PeerMapping* dst);
  static bool cma_disabled_by_param();
  // Unlinks segments left in /dev/shm by processes that no longer exist; returns how many.
  static int collect_stale_segments();
  // Fault injection for tests: drop the next n datagrams of a type on send (host side only).
  void inject_drop(DgramType type, int count);
  uint64_t dropped() const { return dropped_; }
  uint64_t sent() const { return sent_; }
  uint64_t eagain_count() const { return eagain_; }

 private:
  bool probe_cma(PeerMapping* dst);
  std::string name_;
  uint32_t id_;
  int fd_ = -1;
  void* base_ = nullptr;
  size_t bytes_ = 0;
  EpSegmentHdr* hdr_ = nullptr;
  MpscByteRing small_, large_;
  MrTableEntry* mr_table_ = nullptr;
  std::mutex av_mu_;
  std::unordered_map<std::string, std::unique_ptr<PeerMapping>> av_;
  std::mutex mr_mu_;
  std::unordered_map<int, int> drop_;  // DgramType -> remaining drops
  uint64_t dropped_ = 0, sent_ = 0, eagain_ = 0;
};

// Worker threads for large cross-memory writes: one proxy thread copying at memcpy speed is the
// ceiling of the host path, several stripes copied at once are not. Jobs carry a shared status
// word (0 pending, 1 done, negative errno) that the poster polls.
class HostCopyPool {
 public:
  static HostCopyPool& instance();
  // False when the pool is disabled (B200NET_HOST_COPY_THREADS=0) or could not start.
  bool submit(uint32_t pid, uint64_t remote_addr, const void* local, size_t len, std::shared_ptr<std::atomic<int>> status);
  int threads() const { return static_cast<int>(workers_.size()); }
  void shutdown();   // joins the workers; the pool restarts on the next submit
  uint64_t jobs_done() const { return done_.load(); }

 private:
  struct Job {
    uint32_t pid;
    uint64_t remote_addr;
    const void* local;
    size_t len;
    std::shared_ptr<std::atomic<int>> status;
  };
  void run();
  bool start_locked();
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Job> jobs_;
  std::vector<std::thread> workers_;
  bool stop_ = false;
  std::atomic<bool> stop_flag_{false};
  std::atomic<int> queued_{0};
  std::atomic<uint64_t> done_{0};
};

// A named shared-memory window (ctrl mailboxes, GIN signal pages): created by its owner, mapped by
// name by the peer.
class ShmWindow {
 public:
  static std::unique_ptr<ShmWindow> create(const std::string& name, size_t bytes);
  static std::unique_ptr<ShmWindow> open(const std::string& name);
  ~ShmWindow();
  void* data() const { return base_; }
  size_t size() const { return bytes_; }
  const std::string& name() const { return name_; }

 private:
  ShmWindow() = default;
  std::string name_;
  void* base_ = nullptr;
  size_t bytes_ = 0;
  bool owner_ = false;
};

}  // namespace b200net
