#include "b200net/pthread_wrap.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "b200net/param.h"

namespace b200net {

int mutex_init(pthread_mutex_t* m, bool errorcheck) {
  pthread_mutexattr_t attr;
  int rc = pthread_mutexattr_init(&attr);
  if (rc) return rc;
  rc = pthread_mutexattr_settype(&attr, errorcheck ? PTHREAD_MUTEX_ERRORCHECK : PTHREAD_MUTEX_NORMAL);
  if (!rc) rc = pthread_mutex_init(m, &attr);
  pthread_mutexattr_destroy(&attr);
  return rc;
}
int mutex_destroy(pthread_mutex_t* m) { return pthread_mutex_destroy(m); }

[[noreturn]] static void die(const char* what, int rc) {
  fprintf(stderr, "b200net: %s failed: %s\n", what, strerror(rc));
  abort();
}
void mutex_lock(pthread_mutex_t* m) {
  const int rc = pthread_mutex_lock(m);
  if (rc) die("pthread_mutex_lock", rc);
}
void mutex_unlock(pthread_mutex_t* m) {
  const int rc = pthread_mutex_unlock(m);
  if (rc) die("pthread_mutex_unlock", rc);
}

Mutex::Mutex() {
  const int rc = mutex_init(&m_, params().errorcheck_mutex.get());
  if (rc) die("pthread_mutex_init", rc);
}
Mutex::~Mutex() { mutex_destroy(&m_); }

}  // namespace b200net
