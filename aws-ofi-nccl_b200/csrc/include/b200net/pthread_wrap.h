// Mutex wrappers: creation honours ERRORCHECK_MUTEX (error-checking type in debug builds), and
// lock/unlock failures abort with a message instead of being ignored
// (reference: src/nccl_ofi_pthread.cpp, include/nccl_ofi_pthread.h).
#pragma once
#include <pthread.h>
#include "b200net/tsa.h"

namespace b200net {

int mutex_init(pthread_mutex_t* m, bool errorcheck);
int mutex_destroy(pthread_mutex_t* m);
void mutex_lock(pthread_mutex_t* m);
void mutex_unlock(pthread_mutex_t* m);

class TSA_CAPABILITY("mutex") Mutex {
 public:
  Mutex();
  ~Mutex();
  Mutex(const Mutex&) = delete;
  Mutex& operator=(const Mutex&) = delete;
  void lock() TSA_ACQUIRE() { mutex_lock(&m_); }
  void unlock() TSA_RELEASE() { mutex_unlock(&m_); }
  pthread_mutex_t* native() { return &m_; }

 private:
  pthread_mutex_t m_;
};

class TSA_SCOPED_CAPABILITY ScopedLock {
 public:
  explicit ScopedLock(Mutex& m) TSA_ACQUIRE(m) : m_(m) { m_.lock(); }
  ~ScopedLock() TSA_RELEASE() { m_.unlock(); }

 private:
  Mutex& m_;
};

}  // namespace b200net
