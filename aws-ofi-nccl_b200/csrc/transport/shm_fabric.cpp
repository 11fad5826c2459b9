#include "b200net/shm_fabric.h"

#include <dirent.h>
#include <fcntl.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/uio.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <stdexcept>

#include "b200net/log.h"
#include "b200net/math.h"
#include "b200net/param.h"

namespace b200net {

static constexpr uint64_t EP_MAGIC = 0x42323030'4e455431ull;  // "B200NET1"
static std::atomic<uint32_t> g_next_ep_id{0};

// staged write fragment: [FragHdr][bytes]
struct FragHdr {
  uint64_t remote_addr;
  uint32_t len;
  uint32_t pad;
};

bool FabricEndpoint::cma_disabled_by_param() { return params().disable_cma.get(); }

// Segments are named b200net.<pid>.<n> (endpoints) and b200net.mb.<pid>.<n>.<m> (mailboxes); a
// process that dies without running its destructors leaves them behind. Unlink those whose owner
// no longer exists.
int FabricEndpoint::collect_stale_segments() {
  DIR* d = opendir("/dev/shm");
  if (!d) return 0;
  int removed = 0;
  while (dirent* e = readdir(d)) {
    int pid = 0;
    if (sscanf(e->d_name, "b200net.mb.%d.", &pid) != 1 && sscanf(e->d_name, "b200net.%d.", &pid) != 1) continue;
    if (pid <= 0 || pid == static_cast<int>(getpid())) continue;
    if (kill(pid, 0) == 0 || errno != ESRCH) continue;   // alive, or not ours to judge
    const std::string name = std::string("/") + e->d_name;
    if (shm_unlink(name.c_str()) == 0) ++removed;
  }
  closedir(d);
  return removed;
}

FabricEndpoint::FabricEndpoint() : id_(g_next_ep_id.fetch_add(1)) {
  char buf[FAB_EP_NAME_LEN];
  snprintf(buf, sizeof(buf), "/b200net.%d.%u", static_cast<int>(getpid()), id_);
  name_ = buf;
  const size_t small_bytes = MpscByteRing::footprint(FAB_SMALL_CELLS, FAB_SMALL_CELL + sizeof(DgramHdr));
  const size_t large_bytes = MpscByteRing::footprint(FAB_LARGE_CELLS, FAB_LARGE_CELL + sizeof(DgramHdr));
  const size_t hdr_bytes = round_up<size_t>(sizeof(EpSegmentHdr), 64);
  const size_t small_off = hdr_bytes;
  const size_t large_off = round_up<size_t>(small_off + small_bytes, 64);
  const size_t mr_off = round_up<size_t>(large_off + large_bytes, 4096);
  bytes_ = round_up<size_t>(mr_off + FAB_MR_TABLE_SLOTS * sizeof(MrTableEntry), 4096);
  shm_unlink(name_.c_str());  // a stale segment of a dead process with the same pid
  fd_ = shm_open(name_.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd_ < 0) throw std::runtime_error("shm_open(" + name_ + ") failed: " + strerror(errno));
  if (ftruncate(fd_, static_cast<off_t>(bytes_)) != 0) {
    const int e = errno;
    close(fd_);
    shm_unlink(name_.c_str());
    throw std::runtime_error(std::string("ftruncate failed: ") + strerror(e));
  }
  base_ = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd_, 0);
  if (base_ == MAP_FAILED) {
    const int e = errno;
    close(fd_);
    shm_unlink(name_.c_str());
    throw std::runtime_error(std::string("mmap failed: ") + strerror(e));
  }
  hdr_ = new (base_) EpSegmentHdr();
  hdr_->pid = static_cast<uint32_t>(getpid());
  hdr_->ep_id = id_;
  hdr_->small_off = small_off;
  hdr_->large_off = large_off;
  hdr_->mr_table_off = mr_off;
  hdr_->total_bytes = bytes_;
  hdr_->closed.store(0);
  char* b = static_cast<char*>(base_);
  small_ = MpscByteRing::create(b + small_off, FAB_SMALL_CELLS, FAB_SMALL_CELL + sizeof(DgramHdr));
  large_ = MpscByteRing::create(b + large_off, FAB_LARGE_CELLS, FAB_LARGE_CELL + sizeof(DgramHdr));
  mr_table_ = reinterpret_cast<MrTableEntry*>(b + mr_off);
  std::atomic_thread_fence(std::memory_order_release);
  hdr_->magic = EP_MAGIC;  // published last: a peer that sees the magic sees initialised rings
  // host-side fault injection requested through the environment ("type:count,type:count")
  const std::string spec = params().fault_drop.get();
  for (size_t pos = 0; pos < spec.size();) {
    size_t end = spec.find(',', pos);
    if (end == std::string::npos) end = spec.size();
    int type = 0, count = 0;
    if (sscanf(spec.substr(pos, end - pos).c_str(), "%d:%d", &type, &count) == 2 && count > 0)
      inject_drop(static_cast<DgramType>(type), count);
    pos = end + 1;
  }
}

FabricEndpoint::~FabricEndpoint() {
  if (hdr_) hdr_->closed.store(1, std::memory_order_release);
  {
    std::lock_guard<std::mutex> g(av_mu_);
    for (auto& [n, m] : av_)
      if (m->base && m->base != base_) munmap(m->base, m->bytes);
    av_.clear();
  }
  if (base_) munmap(base_, bytes_);
  if (fd_ >= 0) close(fd_);
  shm_unlink(name_.c_str());
}

PeerMapping* FabricEndpoint::av_insert(const std::string& name) {
  std::lock_guard<std::mutex> g(av_mu_);
  auto it = av_.find(name);
  if (it != av_.end()) return it->second.get();
  auto m = std::make_unique<PeerMapping>();
  m->name = name;
  if (name == name_) {
    m->base = base_;
    m->bytes = bytes_;
  } else {
    const int fd = shm_open(name.c_str(), O_RDWR, 0600);
    if (fd < 0) return nullptr;
    struct stat st;
    if (fstat(fd, &st) != 0 || static_cast<size_t>(st.st_size) < sizeof(EpSegmentHdr)) {
      close(fd);
      return nullptr;
    }
    m->bytes = static_cast<size_t>(st.st_size);
    m->base = mmap(nullptr, m->bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (m->base == MAP_FAILED) return nullptr;
  }
  m->hdr = static_cast<EpSegmentHdr*>(m->base);
  if (m->hdr->magic != EP_MAGIC || m->hdr->total_bytes > m->bytes) {
    if (m->base != base_) munmap(m->base, m->bytes);
    return nullptr;
  }
  char* b = static_cast<char*>(m->base);
  m->pid = m->hdr->pid;
  m->small = MpscByteRing::attach(b + m->hdr->small_off);
  m->large = MpscByteRing::attach(b + m->hdr->large_off);
  m->mr_table = reinterpret_cast<MrTableEntry*>(b + m->hdr->mr_table_off);
  PeerMapping* raw = m.get();
  av_[name] = std::move(m);
  return raw;
}

void FabricEndpoint::av_remove(const std::string& name) {
  std::lock_guard<std::mutex> g(av_mu_);
  auto it = av_.find(name);
  if (it == av_.end()) return;
  if (it->second->base && it->second->base != base_) munmap(it->second->base, it->second->bytes);
  av_.erase(it);
}

void FabricEndpoint::inject_drop(DgramType type, int count) { drop_[static_cast<int>(type)] = count; }

int FabricEndpoint::send(PeerMapping* dst, DgramType type, uint16_t flags, const void* a, size_t alen, const void* b,
                         size_t blen) {
  if (!dst) return -EINVAL;
  if (dst->hdr->closed.load(std::memory_order_acquire)) return -ENOTCONN;
  const size_t len = alen + blen;
  if (len > FAB_LARGE_CELL) return -EMSGSIZE;
  if (!drop_.empty()) {
    auto it = drop_.find(static_cast<int>(type));
    if (it != drop_.end() && it->second > 0) {
      --it->second;
      ++dropped_;
      return 0;  // the sender believes it went out
    }
  }
  // header + first fragment are gathered into one contiguous prefix; small on-stack copy
  DgramHdr h{static_cast<uint16_t>(type), flags, id_, static_cast<uint32_t>(getpid()), static_cast<uint32_t>(len)};
  MpscByteRing& ring = (len <= FAB_SMALL_CELL && !(flags & DGRAM_FLAG_ORDER_AFTER_FRAGS)) ? dst->small : dst->large;
  bool ok;
  if (blen == 0) {
    ok = ring.push(&h, sizeof(h), a, alen);
  } else {
    // three fragments: copy header + a into a scratch prefix
    char prefix[sizeof(DgramHdr) + 256];
    if (alen > 256) return -EMSGSIZE;
    memcpy(prefix, &h, sizeof(h));
    memcpy(prefix + sizeof(h), a, alen);
    ok = ring.push(prefix, sizeof(h) + alen, b, blen);
  }
  if (!ok) {
    ++eagain_;
    return -EAGAIN;
  }
  ++sent_;
  return 0;
}

// Cross-memory attach is assumed to work until the kernel refuses it (ptrace policy); the first
// refusal switches this peer to staged writes for good.
bool FabricEndpoint::probe_cma(PeerMapping* dst) {
  if (!dst->cma_probed) {
    dst->cma_probed = true;
    dst->cma_ok = !cma_disabled_by_param();
  }
  return dst->cma_ok;
}

bool FabricEndpoint::writes_are_staged(PeerMapping* dst) {
  if (dst->pid == static_cast<uint32_t>(getpid()) && !cma_disabled_by_param()) return false;
  return !probe_cma(dst);
}

int FabricEndpoint::write_host(PeerMapping* dst, uint64_t remote_addr, const void* local, size_t len, size_t* done) {
  if (!dst || !done) return -EINVAL;
  if (*done >= len) return 0;
  if (dst->hdr->closed.load(std::memory_order_acquire)) return -ENOTCONN;
  if (dst->pid == static_cast<uint32_t>(getpid()) && !cma_disabled_by_param()) {
    memcpy(reinterpret_cast<char*>(remote_addr) + *done, static_cast<const char*>(local) + *done, len - *done);
    *done = len;
    return 0;
  }
  if (probe_cma(dst)) {
    while (*done < len) {
      iovec l{const_cast<char*>(static_cast<const char*>(local)) + *done, len - *done};
      iovec r{reinterpret_cast<void*>(remote_addr + *done), len - *done};
      const ssize_t n = process_vm_writev(static_cast<pid_t>(dst->pid), &l, 1, &r, 1, 0);
      if (n < 0) {
        if (*done == 0 && (errno == EPERM || errno == ENOSYS)) {
          NET_INFO(NCCL_NET, "cross-memory attach to pid %u refused (%s): using staged writes", dst->pid,
                   strerror(errno));
          dst->cma_ok = false;
          break;
        }
        return errno == ESRCH ? -ENOTCONN : -EFAULT;
      }
      *done += static_cast<size_t>(n);
    }
    if (*done >= len) return 0;
  }
  // staged path: fragments that the target applies when it polls; stop at the first full ring
  const size_t chunk = FAB_LARGE_CELL - sizeof(FragHdr);
  while (*done < len) {
    const size_t n = std::min(chunk, len - *done);
    FragHdr fh{remote_addr + *done, static_cast<uint32_t>(n), 0};
    // always through the large ring, however short: the completion that follows travels there too,
    // and only datagrams of one ring are seen in the order they were posted
    const int rc = send(dst, DgramType::WRITE_FRAG, DGRAM_FLAG_ORDER_AFTER_FRAGS, &fh, sizeof(fh),
                        static_cast<const char*>(local) + *done, n);
    if (rc != 0) return rc;  // -EAGAIN: caller retries later from *done
    *done += n;
  }
  return 0;
}

// ------------------------------------------------------------------------------------------ copy workers
HostCopyPool& HostCopyPool::instance() {
  static HostCopyPool* pool = new HostCopyPool();   // never destroyed: workers are joined by shutdown()
  return *pool;
}

bool HostCopyPool::start_locked() {
  if (!workers_.empty()) return true;
  const int n = static_cast<int>(params().host_copy_threads.get());
  if (n <= 0) return false;
  stop_ = false;
  stop_flag_.store(false);
  try {
    for (int i = 0; i < n; ++i) workers_.emplace_back([this] { run(); });
  } catch (const std::exception&) {
    return !workers_.empty();
  }
  return true;
}

bool HostCopyPool::submit(uint32_t pid, uint64_t remote_addr, const void* local, size_t len,
                          std::shared_ptr<std::atomic<int>> status) {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!start_locked()) return false;
    status->store(0, std::memory_order_relaxed);
    jobs_.push_back(Job{pid, remote_addr, local, len, std::move(status)});
    queued_.fetch_add(1, std::memory_order_release);
  }
  cv_.notify_one();
  return true;
}

void HostCopyPool::run() {
  using clock = std::chrono::steady_clock;
  for (;;) {
    Job j;
    bool have = false;
    // Stripes arrive in bursts (one per rail of a chunk, a chunk per channel): poll for a short
    // while before sleeping, so the next stripe does not pay a futex wake-up.
    const auto spin_until = clock::now() + std::chrono::microseconds(100);
    while (!have && clock::now() < spin_until) {
      if (queued_.load(std::memory_order_acquire) > 0) {
        std::lock_guard<std::mutex> g(mu_);
        if (!jobs_.empty()) {
          j = std::move(jobs_.front());
          jobs_.pop_front();
          queued_.fetch_sub(1, std::memory_order_relaxed);
          have = true;
        }
      } else {
#if defined(__x86_64__)
        __builtin_ia32_pause();
#endif
      }
      if (stop_flag_.load(std::memory_order_relaxed)) break;
    }
    if (!have) {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [this] { return stop_ || !jobs_.empty(); });
      if (jobs_.empty()) return;   // stop requested and nothing left
      j = std::move(jobs_.front());
      jobs_.pop_front();
      queued_.fetch_sub(1, std::memory_order_relaxed);
    }
    int result = 1;
    size_t done = 0;
    while (done < j.len) {
      iovec l{const_cast<char*>(static_cast<const char*>(j.local)) + done, j.len - done};
      iovec r{reinterpret_cast<void*>(j.remote_addr + done), j.len - done};
      const ssize_t n = process_vm_writev(static_cast<pid_t>(j.pid), &l, 1, &r, 1, 0);
      if (n <= 0) {
        result = n < 0 ? -errno : -EFAULT;
        break;
      }
      done += static_cast<size_t>(n);
    }
    done_.fetch_add(1, std::memory_order_relaxed);
    j.status->store(result, std::memory_order_release);
  }
}

void HostCopyPool::shutdown() {
  std::vector<std::thread> ws;
  {
    std::lock_guard<std::mutex> g(mu_);
    stop_ = true;
    stop_flag_.store(true);
    ws.swap(workers_);
  }
  cv_.notify_all();
  for (auto& t : ws)
    if (t.joinable()) t.join();
}

int FabricEndpoint::read_host(PeerMapping* dst, uint64_t remote_addr, void* local, size_t len) {
  if (!dst) return -EINVAL;
  if (len == 0) return 0;
  if (dst->pid == static_cast<uint32_t>(getpid())) {
    memcpy(local, reinterpret_cast<const void*>(remote_addr), len);
    return 0;
  }
  if (!probe_cma(dst)) return -ENOTSUP;
  size_t done = 0;
  while (done < len) {
    iovec l{static_cast<char*>(local) + done, len - done};
    iovec r{reinterpret_cast<void*>(remote_addr + done), len - done};
    const ssize_t n = process_vm_readv(static_cast<pid_t>(dst->pid), &l, 1, &r, 1, 0);
    if (n < 0) {
      if (done == 0 && (errno == EPERM || errno == ENOSYS)) {
        dst->cma_ok = false;
        return -ENOTSUP;
      }
      return -EFAULT;
    }
    done += static_cast<size_t>(n);
  }
  return 0;
}

int FabricEndpoint::poll(int budget, const DgramHandler& handler) {
  int n = 0;
  for (MpscByteRing* ring : {&small_, &large_}) {
    while (n < budget) {
      size_t len = 0;
      const void* p = ring->peek(&len);
      if (!p) break;
      const DgramHdr* h = static_cast<const DgramHdr*>(p);
      const char* payload = static_cast<const char*>(p) + sizeof(DgramHdr);
      if (h->type == static_cast<uint16_t>(DgramType::WRITE_FRAG)) {
        const FragHdr* fh = reinterpret_cast<const FragHdr*>(payload);
        memcpy(reinterpret_cast<void*>(fh->remote_addr), payload + sizeof(FragHdr), fh->len);
      } else {
        handler(*h, payload);
      }
      ring->release_front();
      ++n;
    }
  }
  return n;
}

int FabricEndpoint::mr_publish(const MrTableEntry& e) {
  std::lock_guard<std::mutex> g(mr_mu_);
  for (size_t i = 0; i < FAB_MR_TABLE_SLOTS; ++i) {
    const size_t slot = (e.key + i) % FAB_MR_TABLE_SLOTS;
    if (mr_table_[slot].key == 0) {
      MrTableEntry tmp = e;
      tmp.key = 0;
      mr_table_[slot] = tmp;
      std::atomic_thread_fence(std::memory_order_release);
      reinterpret_cast<std::atomic<uint64_t>*>(&mr_table_[slot].key)->store(e.key, std::memory_order_release);
      return 0;
    }
  }
  return -ENOSPC;
}

void FabricEndpoint::mr_unpublish(uint64_t key) {
  std::lock_guard<std::mutex> g(mr_mu_);
  for (size_t i = 0; i < FAB_MR_TABLE_SLOTS; ++i) {
    const size_t slot = (key + i) % FAB_MR_TABLE_SLOTS;
    if (mr_table_[slot].key == key) {
      reinterpret_cast<std::atomic<uint64_t>*>(&mr_table_[slot].key)->store(0, std::memory_order_release);
      return;
    }
  }
}

const MrTableEntry* FabricEndpoint::mr_lookup(const PeerMapping* peer, uint64_t key) {
  if (!peer || key == 0) return nullptr;
  for (size_t i = 0; i < FAB_MR_TABLE_SLOTS; ++i) {
    const size_t slot = (key + i) % FAB_MR_TABLE_SLOTS;
    const uint64_t k = reinterpret_cast<const std::atomic<uint64_t>*>(&peer->mr_table[slot].key)->load(std::memory_order_acquire);
    if (k == key) return &peer->mr_table[slot];
  }
  return nullptr;
}

// ---------------------------------------------------------------- ShmWindow
std::unique_ptr<ShmWindow> ShmWindow::create(const std::string& name, size_t bytes) {
  shm_unlink(name.c_str());
  const int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) return nullptr;
  bytes = round_up<size_t>(bytes, 4096);
  if (ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
    close(fd);
    shm_unlink(name.c_str());
    return nullptr;
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) {
    shm_unlink(name.c_str());
    return nullptr;
  }
  memset(p, 0, bytes);
  std::unique_ptr<ShmWindow> w(new ShmWindow());
  w->name_ = name;
  w->base_ = p;
  w->bytes_ = bytes;
  w->owner_ = true;
  return w;
}

std::unique_ptr<ShmWindow> ShmWindow::open(const std::string& name) {
  const int fd = shm_open(name.c_str(), O_RDWR, 0600);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size <= 0) {
    close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return nullptr;
  std::unique_ptr<ShmWindow> w(new ShmWindow());
  w->name_ = name;
  w->base_ = p;
  w->bytes_ = static_cast<size_t>(st.st_size);
  return w;
}

ShmWindow::~ShmWindow() {
  if (base_) munmap(base_, bytes_);
  if (owner_) shm_unlink(name_.c_str());
}

}  // namespace b200net
