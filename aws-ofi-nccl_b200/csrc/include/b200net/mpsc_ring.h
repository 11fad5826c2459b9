// Bounded multi-producer single-consumer ring (per-cell sequence numbers, CAS on the enqueue
// cursor). All slots are usable. The storage is position independent — no pointers inside —
// so the same ring can be placed in a POSIX shared-memory segment and used between processes
// (reference: include/nccl_ofi_mpsc_ring.h; the cross-process placement is new here).
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <new>
#include "b200net/math.h"

namespace b200net {

// Header + cells laid out contiguously: [MpscRingHdr][cell 0][cell 1]...; cell = {seq, len, payload}.
struct alignas(64) MpscRingHdr {
  uint64_t capacity;    // number of cells, power of two
  uint64_t cell_bytes;  // payload bytes per cell
  alignas(64) std::atomic<uint64_t> enqueue_pos;
  alignas(64) std::atomic<uint64_t> dequeue_pos;
};

class MpscByteRing {
 public:
  static size_t cell_stride(size_t cell_bytes) { return round_up<size_t>(16 + cell_bytes, 64); }
  static size_t footprint(size_t capacity, size_t cell_bytes) {
    return sizeof(MpscRingHdr) + capacity * cell_stride(cell_bytes);
  }
  // Initialise ring storage at `mem` (must be 64-byte aligned and zero or garbage).
  static MpscByteRing create(void* mem, size_t capacity, size_t cell_bytes) {
    auto* h = new (mem) MpscRingHdr();
    h->capacity = capacity;
    h->cell_bytes = cell_bytes;
    h->enqueue_pos.store(0, std::memory_order_relaxed);
    h->dequeue_pos.store(0, std::memory_order_relaxed);
    MpscByteRing r(h);
    for (uint64_t i = 0; i < capacity; ++i) r.seq(i).store(i, std::memory_order_relaxed);
    std::atomic_thread_fence(std::memory_order_release);
    return r;
  }
  static MpscByteRing attach(void* mem) { return MpscByteRing(static_cast<MpscRingHdr*>(mem)); }
  MpscByteRing() = default;

  bool valid() const { return h_ != nullptr; }
  size_t capacity() const { return h_->capacity; }
  size_t cell_bytes() const { return h_->cell_bytes; }

  // Producer side (any thread / process). Two payload fragments are gathered into the cell.
  bool push(const void* a, size_t alen, const void* b = nullptr, size_t blen = 0) {
    if (alen + blen > h_->cell_bytes) return false;
    uint64_t pos = h_->enqueue_pos.load(std::memory_order_relaxed);
    for (;;) {
      const uint64_t s = seq(pos & (h_->capacity - 1)).load(std::memory_order_acquire);
      const int64_t dif = static_cast<int64_t>(s) - static_cast<int64_t>(pos);
      if (dif == 0) {
        if (h_->enqueue_pos.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) break;
      } else if (dif < 0) {
        return false;  // full
      } else {
        pos = h_->enqueue_pos.load(std::memory_order_relaxed);
      }
    }
    const uint64_t idx = pos & (h_->capacity - 1);
    char* c = cell(idx);
    *reinterpret_cast<uint32_t*>(c + 8) = static_cast<uint32_t>(alen + blen);
    if (alen) std::memcpy(c + 16, a, alen);
    if (blen) std::memcpy(c + 16 + alen, b, blen);
    seq(idx).store(pos + 1, std::memory_order_release);
    return true;
  }

  // Consumer side (one thread). Returns a pointer into the ring valid until release_front().
  const void* peek(size_t* len) {
    const uint64_t pos = h_->dequeue_pos.load(std::memory_order_relaxed);
    const uint64_t idx = pos & (h_->capacity - 1);
    if (seq(idx).load(std::memory_order_acquire) != pos + 1) return nullptr;
    char* c = cell(idx);
    if (len) *len = *reinterpret_cast<uint32_t*>(c + 8);
    return c + 16;
  }
  void release_front() {
    const uint64_t pos = h_->dequeue_pos.load(std::memory_order_relaxed);
    const uint64_t idx = pos & (h_->capacity - 1);
    seq(idx).store(pos + h_->capacity, std::memory_order_release);
    h_->dequeue_pos.store(pos + 1, std::memory_order_relaxed);
  }
  bool pop(void* out, size_t out_cap, size_t* len) {
    size_t l = 0;
    const void* p = peek(&l);
    if (!p) return false;
    if (l > out_cap) l = out_cap;
    std::memcpy(out, p, l);
    if (len) *len = l;
    release_front();
    return true;
  }
  bool empty() {
    const uint64_t pos = h_->dequeue_pos.load(std::memory_order_relaxed);
    return seq(pos & (h_->capacity - 1)).load(std::memory_order_acquire) != pos + 1;
  }

 private:
  explicit MpscByteRing(MpscRingHdr* h) : h_(h), stride_(cell_stride(h->cell_bytes)) {}
  char* cell(uint64_t i) { return reinterpret_cast<char*>(h_) + sizeof(MpscRingHdr) + i * stride_; }
  std::atomic<uint64_t>& seq(uint64_t i) { return *reinterpret_cast<std::atomic<uint64_t>*>(cell(i)); }
  MpscRingHdr* h_ = nullptr;
  size_t stride_ = 0;
};

// Typed in-process convenience wrapper owning its storage.
template <typename T>
class MpscRing {
 public:
  explicit MpscRing(size_t capacity = 1024) {
    const size_t cap = next_pow2(capacity);
    mem_ = ::operator new(MpscByteRing::footprint(cap, sizeof(T)), std::align_val_t(64));
    ring_ = MpscByteRing::create(mem_, cap, sizeof(T));
  }
  ~MpscRing() { ::operator delete(mem_, std::align_val_t(64)); }
  MpscRing(const MpscRing&) = delete;
  MpscRing& operator=(const MpscRing&) = delete;
  bool push(const T& v) { return ring_.push(&v, sizeof(T)); }
  bool pop(T& out) { return ring_.pop(&out, sizeof(T), nullptr); }
  bool empty() { return ring_.empty(); }
  size_t capacity() const { return ring_.capacity(); }

 private:
  void* mem_ = nullptr;
  MpscByteRing ring_;
};

}  // namespace b200net
