// Host side of the plugin's own device kernels (copy with completion flag, eager pack): loads the
// embedded sm_100a image into the current CUDA context through the driver shim and hands out
// completion slots in pinned host memory
// (reference: the NIC performs these transfers, src/rdma/nccl_ofi_rdma.cpp post_rdma_write;
//  completions arrive through the CQ, src/rdma/nccl_ofi_rdma.cpp process_completions).
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <mutex>
#include <vector>

#include "b200net/cuda_shim.h"
#include "b200net/idpool.h"

namespace b200net {

class NetKernels {
 public:
  static constexpr int NUM_FLAGS = 1024;
  static constexpr int NUM_EAGER_SLOTS = 64;
  static constexpr size_t EAGER_PAYLOAD_MAX = 8192;
  static constexpr size_t BULK_MIN = 65536;
  static constexpr unsigned BULK_SMEM = 4 * 32768 + 64;   // four pieces and their mbarriers
  static constexpr size_t EAGER_SLOT_BYTES = 16 + EAGER_PAYLOAD_MAX + 8 + 8;  // header, payload, pad, flag

  // The instance of the calling thread's current CUDA context; nullptr when there is no GPU, no
  // context, the image does not load (not an sm_100a device) or B200NET_COPY_KERNEL=0.
  static NetKernels* get();

  // dst[0,n) = src[0,n) on stream `st` with `ctas` CTAs (0 = size based); *slot receives the
  // completion slot to poll with done() and to give back with release(). -EAGAIN: no slot free.
  // 16-byte aligned transfers of at least BULK_MIN bytes go to the bulk-copy kernel (one thread per
  // CTA driving cp.async.bulk through shared memory) unless B200NET_COPY_KERNEL_BULK=0.
  int copy_flag(void* dst, const void* src, size_t n, cuda::Stream st, int ctas, int* slot, bool allow_bulk = true);
  bool done(int slot) const;
  // 0 while the copy runs, 1 when it has completed, -EIO when the kernel gave up on a wait (or its
  // launch failed). Also drives the queue of copy_queue(): a caller that polls its slot needs no
  // other call for its copy to start.
  int status(int slot);
  void release(int slot);

  // The same transfer on the instance's own stream, but the launch waits for company: the transfer
  // is queued, and everything queued leaves in ONE launch of the batch kernel (up to MAX_BATCH
  // transfers, each with its own completion slot) once no further transfer has been queued for
  // B200NET_COPY_BATCH_QUIET_NS (at most B200NET_COPY_BATCH_HOLD_NS after the first) and fewer than
  // B200NET_COPY_BATCH_DEPTH launches are in flight, or the queue is full, or the oldest entry is
  // B200NET_COPY_BATCH_MAX_AGE_US old. A lone message pays the quiet period (1 us).
  // (The reference coalesces the doorbells of consecutive posts with FI_MORE,
  // src/nccl_ofi_rdma.cpp:1876-1919; on this transport the doorbell is a kernel launch.) The launches of a burst of stripes (NCCL posts one per
  // channel) then cost one launch latency per batch instead of one per stripe, serialised on the
  // one stream.
  int copy_queue(void* dst, const void* src, size_t n, int* slot, bool allow_bulk = true);
  // Launches what is due; cheap when nothing is queued. Called from the endpoints' progress loops.
  void poll();
  static constexpr int MAX_BATCH = 16;
  uint64_t batch_launches() const { return batch_launches_.load(); }
  uint64_t batched_jobs() const { return batched_jobs_.load(); }

  // *word += value on the device, release-ordered at system scope (stream-ordered on `st`; the
  // caller synchronises or orders later work on the same stream). -ENOSYS without the kernel.
  int signal_add(void* word, uint64_t value, cuda::Stream st);

  // Packs a device payload (n <= EAGER_PAYLOAD_MAX) and a 16-byte header into a pinned slot.
  int eager_pack(const void* dev_src, size_t n, uint64_t hdr0, uint64_t hdr1, cuda::Stream st, int* slot);
  bool eager_done(int slot) const;
  const uint8_t* eager_slot(int slot) const { return eager_ + static_cast<size_t>(slot) * EAGER_SLOT_BYTES; }
  void eager_release(int slot);

  // The one stream all of the plugin's device work of this context runs on (created with the
  // instance, greatest priority). One stream, not one per rail or endpoint: the device has a
  // handful of hardware work queues that all streams of the process share, and work queued behind
  // a collective kernel in the queue that this work lands in would wait for that kernel, which in
  // turn waits for this work. Every further stream is one more chance to share such a queue.
  cuda::Stream stream() const { return stream_; }

  uint64_t launches() const { return launches_.load(); }

 private:
  NetKernels() = default;
  int init();
  int copy_impl(void* dst, const void* src, size_t n, cuda::Stream st, int ctas, int* slot, bool warm_bulk, bool allow_bulk);
  struct Job {
    void* dst;
    const void* src;
    size_t n;
    int slot;
    uint64_t value;
    bool allow_bulk;
  };
  bool bulk_ok(const Job& j, bool warm = false) const;
  int launch_single(const Job& j, cuda::Stream st, int ctas, bool warm_bulk);
  int flush_locked(bool force);            // lock_ held
  void launched_locked(const Job* jobs, int n);   // bookkeeping of one launch that carries n slots
  void* fn_batch_ = nullptr;
  std::vector<Job> queue_;                 // transfers waiting for their launch (at most MAX_BATCH)
  std::atomic<int> queued_{0};
  uint64_t first_queued_ns_ = 0, last_queued_ns_ = 0;
  int launches_in_flight_ = 0;             // launches with a transfer whose completion word is not set yet
  std::vector<int> slot_launch_;           // slot -> index into launch_remaining_, -1 none (or counted), -2 queued
  std::vector<int> launch_remaining_;      // transfers of that launch not seen complete yet
  std::vector<int> live_slots_;            // launched, completion not counted yet
  void count_slot_locked(int slot);        // the transfer in `slot` is over: one less for its launch
  void reap_locked();                      // counts the live transfers whose completion words are set
  uint64_t launch_seq_ = 0;
  std::atomic<uint64_t> batch_launches_{0}, batched_jobs_{0};
  void* module_ = nullptr;
  void* fn_copy_ = nullptr;
  void* fn_pack_ = nullptr;
  void* fn_signal_ = nullptr;
  cuda::Stream stream_ = nullptr;
  void* fn_bulk_ = nullptr;      // null: not in the image or shared memory cannot be raised
  volatile uint64_t* flags_ = nullptr;   // pinned host, NUM_FLAGS words
  uint32_t* counters_ = nullptr;         // device, NUM_FLAGS words, zero when idle
  uint8_t* eager_ = nullptr;             // pinned host, NUM_EAGER_SLOTS slots
  std::vector<uint64_t> expect_, eager_expect_;
  std::vector<int> free_flags_, free_eager_;
  std::mutex lock_;
  uint64_t next_value_ = 1;
  std::atomic<uint64_t> launches_{0};
};

}  // namespace b200net
