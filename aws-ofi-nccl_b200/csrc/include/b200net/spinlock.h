// Test-and-test-and-set spinlock with pause/isb back-off, annotated for thread-safety analysis
// (reference: include/nccl_ofi_spinlock.h).
#pragma once
#include <atomic>
#include "b200net/tsa.h"

namespace b200net {

inline void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
  __builtin_ia32_pause();
#elif defined(__aarch64__)
  asm volatile("isb" ::: "memory");
#endif
}

class TSA_CAPABILITY("mutex") Spinlock {
 public:
  Spinlock() = default;
  Spinlock(const Spinlock&) = delete;
  Spinlock& operator=(const Spinlock&) = delete;
  void lock() TSA_ACQUIRE() {
    for (;;) {
      if (!flag_.exchange(true, std::memory_order_acquire)) return;
      while (flag_.load(std::memory_order_relaxed)) cpu_relax();
    }
  }
  bool try_lock() TSA_TRY_ACQUIRE(true) {
    return !flag_.load(std::memory_order_relaxed) && !flag_.exchange(true, std::memory_order_acquire);
  }
  void unlock() TSA_RELEASE() { flag_.store(false, std::memory_order_release); }

 private:
  std::atomic<bool> flag_{false};
};

}  // namespace b200net
