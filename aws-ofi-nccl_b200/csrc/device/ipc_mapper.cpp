#include "b200net/ipc_mapper.h"

#include <sys/syscall.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <array>
#include <deque>
#include <map>
#include <mutex>
#include <thread>

namespace b200net {
namespace {

// Queue state lives for the whole process: the helper may be inside the driver when the plugin's
// static destructors run, and a condition variable with a waiter must not be destroyed.
struct Shared {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::shared_ptr<IpcMapJob>> jobs;
  bool started = false;
};
Shared& shared() {
  static Shared* s = new Shared;
  return *s;
}

// Duplicates descriptor `fd` of process `pid` into this process (pidfd_open + pidfd_getfd; the same
// permission as cross-memory attach). Returns the new descriptor or a negative errno.
int steal_fd(uint32_t pid, int fd) {
#if defined(SYS_pidfd_open) && defined(SYS_pidfd_getfd)
  const int pidfd = static_cast<int>(syscall(SYS_pidfd_open, static_cast<pid_t>(pid), 0));
  if (pidfd < 0) return -errno;
  const int mine = static_cast<int>(syscall(SYS_pidfd_getfd, pidfd, fd, 0));
  const int err = errno;
  close(pidfd);
  return mine < 0 ? -err : mine;
#else
  (void)pid;
  (void)fd;
  return -ENOSYS;
#endif
}

int open_vmm(IpcMapJob& job, void** mapped) {
  VmmShare sh;
  memcpy(&sh, job.handle, sizeof(sh));
  if (sh.magic != VMM_SHARE_MAGIC || sh.bytes == 0) return -EINVAL;
  const int fd = steal_fd(sh.pid, sh.fd);
  if (fd < 0) return fd;
  job.bytes = sh.bytes;
  const int rc = cuda::vmm_import_map(fd, sh.bytes, mapped);
  close(fd);   // the imported handle holds its own reference
  return rc;
}

void helper_main() {
  Shared& s = shared();
  for (;;) {
    std::shared_ptr<IpcMapJob> job;
    {
      std::unique_lock<std::mutex> lk(s.mu);
      s.cv.wait(lk, [&] { return !s.jobs.empty(); });
      job = std::move(s.jobs.front());
      s.jobs.pop_front();
    }
    if (job->ctx) cuda::ctx_set_current(job->ctx);
    void* p = nullptr;
    const int rc = job->vmm ? open_vmm(*job, &p) : cuda::ipc_open(job->handle, &p);
    job->mapped = p;
    int expected = 0;
    if (!job->state.compare_exchange_strong(expected, rc == 0 ? 1 : (rc < 0 ? rc : -EIO), std::memory_order_acq_rel) &&
        rc == 0)
      job->close_mapping();   // abandoned meanwhile: nobody is left to use or close it
  }
}

}  // namespace

IpcMapper& IpcMapper::instance() {
  static IpcMapper* m = new IpcMapper;
  return *m;
}

std::shared_ptr<IpcMapJob> IpcMapper::submit(const uint8_t handle[64], cuda::Context ctx, bool vmm) {
  Shared& s = shared();
  auto job = std::make_shared<IpcMapJob>();
  job->vmm = vmm;
  memcpy(job->handle, handle, 64);
  job->ctx = ctx;
  std::lock_guard<std::mutex> g(s.mu);
  if (!s.started) {
    try {
      std::thread(helper_main).detach();
    } catch (...) {
      return nullptr;
    }
    s.started = true;
  }
  s.jobs.push_back(job);
  s.cv.notify_one();
  return job;
}

// Legacy handles opened on the calling thread, shared by everything in this process that names the
// same allocation: the driver does not promise that one handle can be opened twice.
namespace {
struct NowOpen {
  void* mapped;
  int refs;
};
std::mutex g_now_mu;
std::map<std::array<uint8_t, 64>, NowOpen>& now_open() {
  static auto* m = new std::map<std::array<uint8_t, 64>, NowOpen>;
  return *m;
}
}  // namespace

int IpcMapper::open_now(const uint8_t handle[64], bool vmm, void** mapped, size_t* bytes) {
  if (!vmm) {
    *bytes = 0;
    std::array<uint8_t, 64> key;
    memcpy(key.data(), handle, 64);
    std::lock_guard<std::mutex> g(g_now_mu);
    auto it = now_open().find(key);
    if (it != now_open().end()) {
      ++it->second.refs;
      *mapped = it->second.mapped;
      return 0;
    }
    const int rc = cuda::ipc_open(handle, mapped);
    if (rc == 0) now_open()[key] = NowOpen{*mapped, 1};
    return rc;
  }
  IpcMapJob job;
  memcpy(job.handle, handle, 64);
  job.vmm = true;
  const int rc = open_vmm(job, mapped);
  *bytes = job.bytes;
  return rc;
}

int IpcMapper::close_now(void* mapped, bool vmm, size_t bytes) {
  if (vmm) return cuda::vmm_unmap(mapped, bytes);
  {
    std::lock_guard<std::mutex> g(g_now_mu);
    for (auto it = now_open().begin(); it != now_open().end(); ++it) {
      if (it->second.mapped != mapped) continue;
      if (--it->second.refs > 0) return 0;
      now_open().erase(it);
      break;
    }
  }
  return cuda::ipc_close(mapped);
}

int IpcMapper::wait(const IpcMapJob& job, uint64_t wait_us) {
  int st = job.state.load(std::memory_order_acquire);
  if (st != 0 || wait_us == 0) return st;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::microseconds(wait_us);
  while ((st = job.state.load(std::memory_order_acquire)) == 0 && std::chrono::steady_clock::now() < deadline)
    std::this_thread::yield();
  return st;
}

}  // namespace b200net
