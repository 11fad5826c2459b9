// Single-producer single-consumer ring; one slot is kept empty, so capacity-1 items fit
// (reference: include/nccl_ofi_spsc_ring.h).
#pragma once
#include <atomic>
#include <cstddef>
#include <memory>
#include "b200net/math.h"

namespace b200net {

template <typename T>
class SpscRing {
 public:
  explicit SpscRing(size_t capacity_pow2 = 1024) : cap_(next_pow2(capacity_pow2)), buf_(new T[cap_]) {}
  bool push(const T& v) {
    const size_t t = tail_.load(std::memory_order_relaxed);
    const size_t nt = (t + 1) & (cap_ - 1);
    if (nt == head_.load(std::memory_order_acquire)) return false;  // full
    buf_[t] = v;
    tail_.store(nt, std::memory_order_release);
    return true;
  }
  bool pop(T& out) {
    const size_t h = head_.load(std::memory_order_relaxed);
    if (h == tail_.load(std::memory_order_acquire)) return false;  // empty
    out = buf_[h];
    head_.store((h + 1) & (cap_ - 1), std::memory_order_release);
    return true;
  }
  bool empty() const { return head_.load(std::memory_order_acquire) == tail_.load(std::memory_order_acquire); }
  size_t capacity() const { return cap_; }
  size_t usable() const { return cap_ - 1; }

 private:
  const size_t cap_;
  std::unique_ptr<T[]> buf_;
  alignas(64) std::atomic<size_t> head_{0};
  alignas(64) std::atomic<size_t> tail_{0};
};

}  // namespace b200net
