// A stand-in for libcuda.so.1 for CPU tests of the plugin's device-buffer paths. "Device memory"
// is POSIX shared memory, so legacy IPC handles really do map one process's buffer into another;
// copies are memcpy; streams and events complete at once; the two kernels of the plugin's embedded
// image are emulated by name (copy + completion flag, eager pack). Built as libcuda.so.1 into a
// directory of its own and found through LD_LIBRARY_PATH by the tests only.
//
// Fault injection through the environment (read at cuInit):
//   FAKE_CUDA_FAIL_IPC_OPEN=1   cuIpcOpenMemHandle fails (the plugin must fall back to staging)
//   FAKE_CUDA_VMM=1             the tests' device buffers come from the virtual-memory API (create,
//                               reserve, map), as NCCL's own buffers do: no legacy IPC handle, but
//                               the allocation can be exported as a file descriptor
//   FAKE_CUDA_FAIL_VMM_IMPORT=1 importing such a descriptor fails
//   FAKE_CUDA_FAIL_IPC_GET=1    cuIpcGetMemHandle fails, as for allocations of the virtual-memory API
//   FAKE_CUDA_PROTECT=0         device addresses stay readable and writable by host code (default:
//                               they are mapped without access, so a host dereference faults)
//   FAKE_CUDA_IPC_OPEN_DELAY_MS=n cuIpcOpenMemHandle takes n milliseconds (a device that is busy)
//   FAKE_CUDA_LAUNCH_DELAY_US=n kernels and asynchronous copies "finish" n microseconds after the call
//                               that queued them returns (a helper thread performs them in order),
//                               and an event is complete once everything queued before its record
//                               has been performed: completions are asynchronous, as on a device
//   FAKE_CUDA_FAIL_MEMCPY_AFTER=n the n-th cuMemcpyAsync from now on and every later one fails
//   (fake_cuda_fail_launch_after(n), a function tests call: the same for cuLaunchKernel)
//   FAKE_CUDA_SUBALLOC_MAX=n    cuMemAlloc requests below n bytes (default 65536) are carved at
//                               256-byte granularity out of shared 2 MiB blocks, as the driver does
//                               with small allocations: several allocations share a page, an IPC
//                               handle names the block plus the offset, and a peer that opens it may
//                               touch only the bytes of that one allocation (anything else aborts)
#include <cuda.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>

#include "b200net/net_kernel_args.h"

namespace {

struct Alloc {
  size_t size;
  std::string shm_name;   // empty: mapping of a peer's allocation
  bool opened_from_peer;
  unsigned char* shadow;   // readable and writable view of the same pages (the device's own view)
  unsigned long long vmm_handle = 0;   // non-zero: mapped through the virtual-memory API
  // carved out of a shared block (own small allocations), or a window into a peer's block:
  int block = -1;              // own: index into g_blocks
  size_t block_off = 0;        // offset of this allocation inside the block
  void* map_base = nullptr;    // peer window: what to unmap on close (the whole block was mapped)
  unsigned char* map_shadow = nullptr;
  size_t map_size = 0;
};
// A 2 MiB shared segment that small allocations are carved from.
struct Block {
  std::string shm_name;
  unsigned char* user = nullptr;     // PROT_NONE view (addresses handed to the program)
  unsigned char* shadow = nullptr;
  std::map<size_t, size_t> used;     // offset -> bytes
};
constexpr size_t kBlockBytes = 2u << 20;
constexpr size_t kSubGranule = 256;
std::mutex g_mu;
std::map<uintptr_t, Alloc> g_allocs;   // base -> allocation ("device" address ranges of this process)
std::map<int, Block> g_blocks;          // guarded by g_mu
int g_next_block = 0;
std::atomic<int> g_next_alloc{0};
std::atomic<long> g_memcpy_budget{-1};  // < 0: copies never fail
std::atomic<long> g_launch_budget{-1};  // < 0: kernel launches never fail
bool g_fail_ipc_open = false;
int g_launch_delay_us = 0;

const Alloc* find_alloc(uintptr_t p, uintptr_t* base) {
  auto it = g_allocs.upper_bound(p);
  if (it == g_allocs.begin()) return nullptr;
  --it;
  if (p >= it->first && p < it->first + it->second.size) {
    *base = it->first;
    return &it->second;
  }
  return nullptr;
}

// "Device" addresses handed to the program are mapped without access rights, so host code that
// dereferences one faults at once, as it would on a real device without unified addressing. The
// stand-in itself (copies, "kernels") works on a second, accessible mapping of the same pages.
// Host addresses pass through unchanged. FAKE_CUDA_PROTECT=0 switches the protection off.
bool protect_on() {
  static const bool on = !(getenv("FAKE_CUDA_PROTECT") && !atoi(getenv("FAKE_CUDA_PROTECT")));
  return on;
}
void* dev_view(const void* p, size_t n = 0) {
  std::lock_guard<std::mutex> g(g_mu);
  uintptr_t base = 0;
  const Alloc* al = find_alloc(reinterpret_cast<uintptr_t>(p), &base);
  if (!al) return const_cast<void*>(p);
  const size_t off = reinterpret_cast<uintptr_t>(p) - base;
  if (off + n > al->size) {
    // a real device would write into a neighbour's bytes (or fault): never let that pass
    fprintf(stderr, "fake libcuda: access of %zu bytes at offset %zu runs past an allocation of %zu bytes\n", n, off, al->size);
    abort();
  }
  return al->shadow + off;
}
// Maps the pages of fd twice: the program's (protected) address and the stand-in's own view.
bool map_pair(int fd, size_t bytes, void** user, unsigned char** shadow) {
  void* u = mmap(nullptr, bytes, protect_on() ? PROT_NONE : (PROT_READ | PROT_WRITE), MAP_SHARED, fd, 0);
  if (u == MAP_FAILED) return false;
  void* sh = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (sh == MAP_FAILED) {
    munmap(u, bytes);
    return false;
  }
  *user = u;
  *shadow = static_cast<unsigned char*>(sh);
  return true;
}

struct IpcHandlePayload {   // fits the 64 opaque bytes
  char name[40];
  uint64_t size;      // of the segment to map
  uint64_t offset;    // of the allocation inside it (small allocations share a block)
  uint64_t bytes;     // of the allocation
};
static_assert(sizeof(IpcHandlePayload) <= sizeof(CUipcMemHandle), "handle payload too large");

// ---- a worker that performs "kernels" after a delay. The queue state is allocated once and never
// destroyed: the worker outlives main(), and destroying a condition variable that a thread still
// waits on blocks the exiting process.
using WorkQueue = std::deque<std::pair<std::chrono::steady_clock::time_point, std::function<void()>>>;
std::mutex& g_wmu = *new std::mutex;
std::condition_variable& g_wcv = *new std::condition_variable;
WorkQueue& g_work = *new WorkQueue;
std::thread* g_worker = nullptr;
std::atomic<int> g_outstanding{0};   // queued or running
// Work handed to the delayed worker is numbered; an event remembers the number current when it was
// recorded and is complete once the worker has passed it.
std::atomic<unsigned long long> g_submitted{0}, g_performed{0};
void worker_main() {
  for (;;) {
    std::function<void()> fn;
    {
      std::unique_lock<std::mutex> lk(g_wmu);
      g_wcv.wait(lk, [] { return !g_work.empty(); });
      auto due = g_work.front().first;
      if (std::chrono::steady_clock::now() < due) {
        lk.unlock();
        std::this_thread::sleep_until(due);
        continue;
      }
      fn = std::move(g_work.front().second);
      g_work.pop_front();
    }
    fn();
    g_performed.fetch_add(1);
    g_outstanding.fetch_sub(1);
  }
}
void run_later(std::function<void()> fn) {
  if (g_launch_delay_us <= 0) {
    fn();
    g_submitted.fetch_add(1);
    g_performed.fetch_add(1);
    return;
  }
  std::lock_guard<std::mutex> g(g_wmu);
  if (!g_worker) g_worker = new std::thread(worker_main);   // lives until the process exits
  g_outstanding.fetch_add(1);
  g_submitted.fetch_add(1);
  g_work.emplace_back(std::chrono::steady_clock::now() + std::chrono::microseconds(g_launch_delay_us), std::move(fn));
  g_wcv.notify_one();
}

enum FakeFn : uintptr_t { FN_COPY_FLAG = 0x101, FN_EAGER_PACK = 0x102, FN_COPY_BULK = 0x103, FN_SIGNAL_ADD = 0x104, FN_COPY_BATCH = 0x105 };

// ------------------------------------------------------------------------------------------ entry points
CUresult fInit(unsigned) {
  g_fail_ipc_open = getenv("FAKE_CUDA_FAIL_IPC_OPEN") && atoi(getenv("FAKE_CUDA_FAIL_IPC_OPEN"));
  g_launch_delay_us = getenv("FAKE_CUDA_LAUNCH_DELAY_US") ? atoi(getenv("FAKE_CUDA_LAUNCH_DELAY_US")) : 0;
  if (const char* v = getenv("FAKE_CUDA_FAIL_MEMCPY_AFTER")) g_memcpy_budget.store(atol(v));
  return CUDA_SUCCESS;
}
CUresult fDeviceGetCount(int* n) {
  *n = getenv("FAKE_CUDA_DEVICES") ? atoi(getenv("FAKE_CUDA_DEVICES")) : 2;
  return CUDA_SUCCESS;
}
CUresult fDeviceGet(CUdevice* d, int ord) {
  *d = ord;
  return CUDA_SUCCESS;
}
CUresult fDeviceGetAttribute(int* v, CUdevice_attribute a, CUdevice) {
  switch (a) {
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR: *v = 10; break;
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR: *v = 0; break;
    case CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT: *v = 148; break;
    case CU_DEVICE_ATTRIBUTE_UNIFIED_ADDRESSING: *v = 1; break;
    default: *v = 0; break;   // no dma-buf, no multicast, no VMM handle types
  }
  return CUDA_SUCCESS;
}
CUresult fDeviceGetP2PAttribute(int* v, CUdevice_P2PAttribute, CUdevice, CUdevice) {
  *v = 1;
  return CUDA_SUCCESS;
}
CUresult fDeviceGetPCIBusId(char* out, int len, CUdevice d) {
  snprintf(out, static_cast<size_t>(len), "0000:%02x:00.0", 0x10 + d);
  return CUDA_SUCCESS;
}
CUresult fDeviceGetUuid(CUuuid* u, CUdevice d) {
  memset(u, 0, sizeof(*u));
  u->bytes[0] = static_cast<char>(0xFA);
  u->bytes[15] = static_cast<char>(d);
  return CUDA_SUCCESS;
}
std::map<uintptr_t, size_t> g_pinned;   // page-locked host ranges (guarded by g_mu)
CUresult fPointerGetAttribute(void* out, CUpointer_attribute a, CUdeviceptr p) {
  std::lock_guard<std::mutex> g(g_mu);
  if (a == CU_POINTER_ATTRIBUTE_DEVICE_POINTER) {
    // page-locked host memory is readable by kernels at its own address; pageable memory is not
    auto it = g_pinned.upper_bound(static_cast<uintptr_t>(p));
    if (it != g_pinned.begin()) {
      --it;
      if (p >= it->first && p < it->first + it->second) {
        *static_cast<CUdeviceptr*>(out) = p;
        return CUDA_SUCCESS;
      }
    }
    uintptr_t b = 0;
    if (find_alloc(static_cast<uintptr_t>(p), &b)) {
      *static_cast<CUdeviceptr*>(out) = p;
      return CUDA_SUCCESS;
    }
    return CUDA_ERROR_INVALID_VALUE;
  }
  uintptr_t base = 0;
  const Alloc* al = find_alloc(static_cast<uintptr_t>(p), &base);
  if (!al) return CUDA_ERROR_INVALID_VALUE;   // what the driver answers for plain host memory
  switch (a) {
    case CU_POINTER_ATTRIBUTE_MEMORY_TYPE: *static_cast<unsigned*>(out) = CU_MEMORYTYPE_DEVICE; break;
    case CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL: *static_cast<int*>(out) = 0; break;
    case CU_POINTER_ATTRIBUTE_IS_LEGACY_CUDA_IPC_CAPABLE: *static_cast<int*>(out) = (al->opened_from_peer || al->vmm_handle) ? 0 : 1; break;
    default: return CUDA_ERROR_INVALID_VALUE;
  }
  return CUDA_SUCCESS;
}
CUresult fMemGetAddressRange(CUdeviceptr* base_out, size_t* size_out, CUdeviceptr p) {
  std::lock_guard<std::mutex> g(g_mu);
  uintptr_t base = 0;
  const Alloc* al = find_alloc(static_cast<uintptr_t>(p), &base);
  if (!al) return CUDA_ERROR_INVALID_VALUE;
  if (base_out) *base_out = base;
  if (size_out) *size_out = al->size;
  return CUDA_SUCCESS;
}
size_t suballoc_max() {
  static const size_t v = getenv("FAKE_CUDA_SUBALLOC_MAX") ? strtoull(getenv("FAKE_CUDA_SUBALLOC_MAX"), nullptr, 0) : 65536;
  return v;
}
// A small allocation: first fit at 256-byte granularity inside a shared block. g_mu is held.
bool carve_locked(size_t bytes, CUdeviceptr* out) {
  const size_t need = (bytes + kSubGranule - 1) & ~(kSubGranule - 1);
  for (int pass = 0; pass < 2; ++pass) {
    for (auto& [id, b] : g_blocks) {
      size_t at = 0;
      for (const auto& [off, len] : b.used) {
        if (off - at >= need) break;
        at = off + ((len + kSubGranule - 1) & ~(kSubGranule - 1));
      }
      if (at + need > kBlockBytes) continue;
      b.used[at] = bytes;
      Alloc al{bytes, b.shm_name, false, b.shadow + at};
      al.block = id;
      al.block_off = at;
      g_allocs[reinterpret_cast<uintptr_t>(b.user + at)] = al;
      *out = reinterpret_cast<CUdeviceptr>(b.user + at);
      return true;
    }
    if (pass == 1) break;
    // no block has room: make one
    char name[40];
    snprintf(name, sizeof(name), "/fakecuda.%d.b%d", static_cast<int>(getpid()), g_next_block);
    shm_unlink(name);
    const int fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) return false;
    void* user = nullptr;
    unsigned char* shadow = nullptr;
    const bool ok = ftruncate(fd, static_cast<off_t>(kBlockBytes)) == 0 && map_pair(fd, kBlockBytes, &user, &shadow);
    close(fd);
    if (!ok) {
      shm_unlink(name);
      return false;
    }
    Block b;
    b.shm_name = name;
    b.user = static_cast<unsigned char*>(user);
    b.shadow = shadow;
    g_blocks[g_next_block++] = std::move(b);
  }
  return false;
}
CUresult fMemAlloc(CUdeviceptr* out, size_t bytes) {
  if (bytes == 0) return CUDA_ERROR_INVALID_VALUE;
  if (bytes < suballoc_max()) {
    std::lock_guard<std::mutex> g(g_mu);
    return carve_locked(bytes, out) ? CUDA_SUCCESS : CUDA_ERROR_OUT_OF_MEMORY;
  }
  char name[40];
  snprintf(name, sizeof(name), "/fakecuda.%d.%d", static_cast<int>(getpid()), g_next_alloc.fetch_add(1));
  shm_unlink(name);
  const int fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) return CUDA_ERROR_OUT_OF_MEMORY;
  const size_t rounded = (bytes + 4095) & ~static_cast<size_t>(4095);
  if (ftruncate(fd, static_cast<off_t>(rounded)) != 0) {
    close(fd);
    shm_unlink(name);
    return CUDA_ERROR_OUT_OF_MEMORY;
  }
  void* p = nullptr;
  unsigned char* shadow = nullptr;
  const bool mapped = map_pair(fd, rounded, &p, &shadow);
  close(fd);
  if (!mapped) {
    shm_unlink(name);
    return CUDA_ERROR_OUT_OF_MEMORY;
  }
  std::lock_guard<std::mutex> g(g_mu);
  Alloc al{bytes, name, false, shadow};
  al.map_size = rounded;
  g_allocs[reinterpret_cast<uintptr_t>(p)] = al;
  *out = reinterpret_cast<CUdeviceptr>(p);
  return CUDA_SUCCESS;
}
CUresult fMemFree(CUdeviceptr p) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_allocs.find(static_cast<uintptr_t>(p));
  if (it == g_allocs.end() || it->second.opened_from_peer) return CUDA_ERROR_INVALID_VALUE;
  if (it->second.block >= 0) {
    auto b = g_blocks.find(it->second.block);
    if (b != g_blocks.end()) {
      b->second.used.erase(it->second.block_off);
      if (b->second.used.empty()) {   // the last allocation of the block: the block goes too
        munmap(b->second.user, kBlockBytes);
        munmap(b->second.shadow, kBlockBytes);
        shm_unlink(b->second.shm_name.c_str());
        g_blocks.erase(b);
      }
    }
    g_allocs.erase(it);
    return CUDA_SUCCESS;
  }
  munmap(reinterpret_cast<void*>(it->first), it->second.map_size);
  munmap(it->second.shadow, it->second.map_size);
  if (!it->second.shm_name.empty()) shm_unlink(it->second.shm_name.c_str());
  g_allocs.erase(it);
  return CUDA_SUCCESS;
}
CUresult fMemsetD8(CUdeviceptr p, unsigned char v, size_t n) {
  memset(dev_view(reinterpret_cast<void*>(p), n), v, n);
  return CUDA_SUCCESS;
}
CUresult fIpcGetMemHandle(CUipcMemHandle* h, CUdeviceptr p) {
  // what the driver answers for memory that came from the virtual-memory API (cuMemCreate)
  if (getenv("FAKE_CUDA_FAIL_IPC_GET") && atoi(getenv("FAKE_CUDA_FAIL_IPC_GET"))) return CUDA_ERROR_INVALID_VALUE;
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_allocs.find(static_cast<uintptr_t>(p));
  if (it == g_allocs.end() || it->second.shm_name.empty()) return CUDA_ERROR_INVALID_VALUE;
  IpcHandlePayload pl{};
  snprintf(pl.name, sizeof(pl.name), "%s", it->second.shm_name.c_str());
  pl.size = it->second.block >= 0 ? kBlockBytes : it->second.map_size;
  pl.offset = it->second.block >= 0 ? it->second.block_off : 0;
  pl.bytes = it->second.size;
  memset(h, 0, sizeof(*h));
  memcpy(h, &pl, sizeof(pl));
  return CUDA_SUCCESS;
}
CUresult fIpcOpenMemHandle(CUdeviceptr* out, CUipcMemHandle h, unsigned) {
  if (g_fail_ipc_open) return CUDA_ERROR_INVALID_DEVICE;
  if (const char* d = getenv("FAKE_CUDA_IPC_OPEN_DELAY_MS")) usleep(1000 * static_cast<useconds_t>(atoi(d)));
  IpcHandlePayload pl;
  memcpy(&pl, &h, sizeof(pl));
  pl.name[sizeof(pl.name) - 1] = 0;
  const int fd = shm_open(pl.name, O_RDWR, 0600);
  if (fd < 0) return CUDA_ERROR_INVALID_VALUE;
  void* p = nullptr;
  unsigned char* shadow = nullptr;
  const bool mapped = map_pair(fd, pl.size, &p, &shadow);
  close(fd);
  if (!mapped) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> g(g_mu);
  // the pointer handed back stands for the allocation the handle was taken from, and only its
  // bytes are reachable through it, although the whole segment is mapped behind it
  Alloc al{pl.bytes, "", true, shadow + pl.offset};
  al.map_base = p;
  al.map_shadow = shadow;
  al.map_size = pl.size;
  g_allocs[reinterpret_cast<uintptr_t>(p) + pl.offset] = al;
  *out = reinterpret_cast<CUdeviceptr>(p) + pl.offset;
  return CUDA_SUCCESS;
}
CUresult fIpcCloseMemHandle(CUdeviceptr p) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_allocs.find(static_cast<uintptr_t>(p));
  if (it == g_allocs.end() || !it->second.opened_from_peer) return CUDA_ERROR_INVALID_VALUE;
  munmap(it->second.map_base, it->second.map_size);
  munmap(it->second.map_shadow, it->second.map_size);
  g_allocs.erase(it);
  return CUDA_SUCCESS;
}
CUresult fCtxGetCurrent(CUcontext* c) {
  *c = reinterpret_cast<CUcontext>(0x1);
  return CUDA_SUCCESS;
}
CUresult fCtxSetCurrent(CUcontext) { return CUDA_SUCCESS; }
CUresult fDevicePrimaryCtxRetain(CUcontext* c, CUdevice) {
  *c = reinterpret_cast<CUcontext>(0x1);
  return CUDA_SUCCESS;
}
CUresult fStreamCreate(CUstream* s, unsigned) {
  static std::atomic<uintptr_t> next{0x1000};
  *s = reinterpret_cast<CUstream>(next.fetch_add(16));
  return CUDA_SUCCESS;
}
CUresult fStreamDestroy(CUstream) { return CUDA_SUCCESS; }
CUresult fStreamSynchronize(CUstream) {
  // delayed work is not tied to streams: wait until none is queued or running
  while (g_outstanding.load() > 0) usleep(50);
  return CUDA_SUCCESS;
}
CUresult fEventCreate(CUevent* e, unsigned) {
  *e = reinterpret_cast<CUevent>(new std::atomic<unsigned long long>(0));
  return CUDA_SUCCESS;
}
CUresult fEventDestroy(CUevent e) {
  delete reinterpret_cast<std::atomic<unsigned long long>*>(e);
  return CUDA_SUCCESS;
}
CUresult fEventRecord(CUevent e, CUstream) {
  reinterpret_cast<std::atomic<unsigned long long>*>(e)->store(g_submitted.load());
  return CUDA_SUCCESS;
}
CUresult fEventQuery(CUevent e) {
  return g_performed.load() >= reinterpret_cast<std::atomic<unsigned long long>*>(e)->load() ? CUDA_SUCCESS : CUDA_ERROR_NOT_READY;
}
CUresult fMemcpyAsync(CUdeviceptr d, CUdeviceptr s, size_t n, CUstream) {
  if (g_memcpy_budget.load() >= 0 && g_memcpy_budget.fetch_sub(1) <= 0) {
    g_memcpy_budget.store(0);
    return CUDA_ERROR_INVALID_VALUE;
  }
  void* to = dev_view(reinterpret_cast<void*>(d), n);
  const void* from = dev_view(reinterpret_cast<const void*>(s), n);
  run_later([=] {
    if (n == 8 && reinterpret_cast<uintptr_t>(to) % 8 == 0 && reinterpret_cast<uintptr_t>(from) % 8 == 0) {
      // an aligned word (a signal): one indivisible store, as the copy engine does it, so that a
      // reader polling the word with an atomic load is not a data race in the eyes of a race detector
      __atomic_store_n(static_cast<unsigned long long*>(to), __atomic_load_n(static_cast<const unsigned long long*>(from), __ATOMIC_ACQUIRE),
                       __ATOMIC_RELEASE);
      return;
    }
    memcpy(to, from, n);
  });
  return CUDA_SUCCESS;
}
CUresult fModuleLoadData(CUmodule* m, const void* image) {
  if (!image) return CUDA_ERROR_INVALID_IMAGE;
  *m = reinterpret_cast<CUmodule>(0x2);
  return CUDA_SUCCESS;
}
CUresult fModuleUnload(CUmodule) { return CUDA_SUCCESS; }
CUresult fFuncSetAttribute(CUfunction, CUfunction_attribute, int) { return CUDA_SUCCESS; }
CUresult fModuleGetFunction(CUfunction* f, CUmodule, const char* name) {
  if (!strcmp(name, "b200net_copy_flag")) *f = reinterpret_cast<CUfunction>(FN_COPY_FLAG);
  else if (!strcmp(name, "b200net_eager_pack")) *f = reinterpret_cast<CUfunction>(FN_EAGER_PACK);
  else if (!strcmp(name, "b200net_copy_bulk")) *f = reinterpret_cast<CUfunction>(FN_COPY_BULK);
  else if (!strcmp(name, "b200net_signal_add")) *f = reinterpret_cast<CUfunction>(FN_SIGNAL_ADD);
  else if (!strcmp(name, "b200net_copy_batch")) *f = reinterpret_cast<CUfunction>(FN_COPY_BATCH);
  else return CUDA_ERROR_NOT_FOUND;
  return CUDA_SUCCESS;
}
CUresult fLaunchKernel(CUfunction f, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void** args,
                       void**) {
  const uintptr_t id = reinterpret_cast<uintptr_t>(f);
  if (g_launch_budget.load() >= 0 && g_launch_budget.fetch_sub(1) <= 0) {
    g_launch_budget.store(0);
    return CUDA_ERROR_LAUNCH_FAILED;
  }
  if (id == FN_COPY_FLAG || id == FN_COPY_BULK) {
    auto* dst = *static_cast<unsigned char**>(args[0]);
    auto* src = *static_cast<const unsigned char**>(args[1]);
    const unsigned long long bytes = *static_cast<unsigned long long*>(args[2]);
    auto* flag = *static_cast<unsigned long long**>(args[4]);
    const unsigned long long value = *static_cast<unsigned long long*>(args[5]);
    run_later([=] {
      memcpy(dev_view(dst, bytes), dev_view(src, bytes), bytes);
      __atomic_store_n(static_cast<unsigned long long*>(dev_view(flag)), value, __ATOMIC_RELEASE);
    });
    return CUDA_SUCCESS;
  }
  if (id == FN_COPY_BATCH) {
    const B200NetBatchArgs a = *static_cast<const B200NetBatchArgs*>(args[0]);
    run_later([=] {
      for (unsigned j = 0; j < a.njobs; ++j) {
        const B200NetBatchJob& job = a.job[j];
        memcpy(dev_view(job.dst, job.bytes), dev_view(job.src, job.bytes), job.bytes);
        __atomic_store_n(static_cast<unsigned long long*>(dev_view(job.flag)), job.flag_value, __ATOMIC_RELEASE);
      }
    });
    return CUDA_SUCCESS;
  }
  if (id == FN_SIGNAL_ADD) {
    auto* word = *static_cast<unsigned long long**>(args[0]);
    const unsigned long long value = *static_cast<unsigned long long*>(args[1]);
    run_later([=] { __atomic_fetch_add(static_cast<unsigned long long*>(dev_view(word, 8)), value, __ATOMIC_ACQ_REL); });
    return CUDA_SUCCESS;
  }
  if (id == FN_EAGER_PACK) {
    auto* slot = *static_cast<unsigned char**>(args[0]);
    auto* payload = *static_cast<const unsigned char**>(args[1]);
    const unsigned bytes = *static_cast<unsigned*>(args[2]);
    const unsigned long long h0 = *static_cast<unsigned long long*>(args[3]);
    const unsigned long long h1 = *static_cast<unsigned long long*>(args[4]);
    const unsigned flag_off = *static_cast<unsigned*>(args[5]);
    const unsigned long long value = *static_cast<unsigned long long*>(args[6]);
    run_later([=] {
      auto* out = static_cast<unsigned char*>(dev_view(slot));
      memcpy(out + 16, dev_view(payload, bytes), bytes);
      memcpy(out, &h0, 8);
      memcpy(out + 8, &h1, 8);
      __atomic_store_n(reinterpret_cast<unsigned long long*>(out + flag_off), value, __ATOMIC_RELEASE);
    });
    return CUDA_SUCCESS;
  }
  return CUDA_ERROR_INVALID_HANDLE;
}
CUresult fMemHostAlloc(void** p, size_t bytes, unsigned) {
  const size_t rounded = (bytes + 4095) & ~static_cast<size_t>(4095);
  if (posix_memalign(p, 4096, rounded) != 0) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> g(g_mu);
  g_pinned[reinterpret_cast<uintptr_t>(*p)] = rounded;
  return CUDA_SUCCESS;
}
CUresult fMemFreeHost(void* p) {
  {
    std::lock_guard<std::mutex> g(g_mu);
    g_pinned.erase(reinterpret_cast<uintptr_t>(p));
  }
  free(p);
  return CUDA_SUCCESS;
}
CUresult fMemHostRegister(void* p, size_t bytes, unsigned) {
  std::lock_guard<std::mutex> g(g_mu);
  g_pinned[reinterpret_cast<uintptr_t>(p)] = bytes;
  return CUDA_SUCCESS;
}
CUresult fMemHostUnregister(void* p) {
  std::lock_guard<std::mutex> g(g_mu);
  g_pinned.erase(reinterpret_cast<uintptr_t>(p));
  return CUDA_SUCCESS;
}
CUresult fCtxSynchronize() {
  while (g_outstanding.load() > 0) usleep(50);
  return CUDA_SUCCESS;
}
// ---- the virtual-memory API: an allocation is a memory file, a handle a reference to it
struct VmmHandle {
  int fd;
  size_t size;
  int refs;
  bool imported;
};
std::map<unsigned long long, VmmHandle> g_handles;   // guarded by g_mu
unsigned long long g_next_handle = 0x7000;

CUresult fMemGetAllocationGranularity(size_t* gran, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) {
  *gran = 65536;
  return CUDA_SUCCESS;
}
CUresult fMemCreate(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp*, unsigned long long) {
  const int fd = memfd_create("fakecuda-vmm", 0);
  if (fd < 0 || ftruncate(fd, static_cast<off_t>(size)) != 0) {
    if (fd >= 0) close(fd);
    return CUDA_ERROR_OUT_OF_MEMORY;
  }
  std::lock_guard<std::mutex> g(g_mu);
  *h = g_next_handle++;
  g_handles[*h] = VmmHandle{fd, size, 1, false};
  return CUDA_SUCCESS;
}
CUresult fMemRelease(CUmemGenericAllocationHandle h) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_handles.find(h);
  if (it == g_handles.end()) return CUDA_ERROR_INVALID_VALUE;
  if (--it->second.refs == 0) {
    close(it->second.fd);
    g_handles.erase(it);
  }
  return CUDA_SUCCESS;
}
CUresult fMemAddressReserve(CUdeviceptr* va, size_t size, size_t, CUdeviceptr, unsigned long long) {
  void* p = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (p == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  *va = reinterpret_cast<CUdeviceptr>(p);
  return CUDA_SUCCESS;
}
CUresult fMemAddressFree(CUdeviceptr va, size_t size) {
  munmap(reinterpret_cast<void*>(va), size);
  return CUDA_SUCCESS;
}
CUresult fMemMap(CUdeviceptr va, size_t size, size_t offset, CUmemGenericAllocationHandle h, unsigned long long) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_handles.find(h);
  if (it == g_handles.end() || offset + size > it->second.size) return CUDA_ERROR_INVALID_VALUE;
  void* user = mmap(reinterpret_cast<void*>(va), size, protect_on() ? PROT_NONE : (PROT_READ | PROT_WRITE), MAP_SHARED | MAP_FIXED,
                    it->second.fd, static_cast<off_t>(offset));
  if (user == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  void* sh = mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_SHARED, it->second.fd, static_cast<off_t>(offset));
  if (sh == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  ++it->second.refs;   // a mapping keeps the allocation alive
  Alloc al{size, "", it->second.imported, static_cast<unsigned char*>(sh)};
  al.vmm_handle = h;
  g_allocs[static_cast<uintptr_t>(va)] = al;
  return CUDA_SUCCESS;
}
CUresult fMemUnmap(CUdeviceptr va, size_t size) {
  unsigned long long h = 0;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_allocs.find(static_cast<uintptr_t>(va));
    if (it == g_allocs.end() || !it->second.vmm_handle || it->second.size != size) return CUDA_ERROR_INVALID_VALUE;
    munmap(it->second.shadow, size);
    h = it->second.vmm_handle;
    g_allocs.erase(it);
  }
  // the address range stays reserved, without backing
  mmap(reinterpret_cast<void*>(va), size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
  return fMemRelease(h);
}
CUresult fMemSetAccess(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) { return CUDA_SUCCESS; }
CUresult fMemRetainAllocationHandle(CUmemGenericAllocationHandle* h, void* addr) {
  std::lock_guard<std::mutex> g(g_mu);
  uintptr_t base = 0;
  const Alloc* al = find_alloc(reinterpret_cast<uintptr_t>(addr), &base);
  if (!al || !al->vmm_handle) return CUDA_ERROR_INVALID_VALUE;
  *h = al->vmm_handle;
  ++g_handles[*h].refs;
  return CUDA_SUCCESS;
}
CUresult fMemExportToShareableHandle(void* out, CUmemGenericAllocationHandle h, CUmemAllocationHandleType type, unsigned long long) {
  if (type != CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) return CUDA_ERROR_NOT_SUPPORTED;
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_handles.find(h);
  if (it == g_handles.end()) return CUDA_ERROR_INVALID_VALUE;
  const int fd = dup(it->second.fd);
  if (fd < 0) return CUDA_ERROR_OUT_OF_MEMORY;
  *static_cast<int*>(out) = fd;
  return CUDA_SUCCESS;
}
CUresult fMemImportFromShareableHandle(CUmemGenericAllocationHandle* h, void* os_handle, CUmemAllocationHandleType type) {
  if (type != CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) return CUDA_ERROR_NOT_SUPPORTED;
  if (getenv("FAKE_CUDA_FAIL_VMM_IMPORT") && atoi(getenv("FAKE_CUDA_FAIL_VMM_IMPORT"))) return CUDA_ERROR_INVALID_DEVICE;
  const int fd = dup(static_cast<int>(reinterpret_cast<uintptr_t>(os_handle)));
  struct stat st;
  if (fd < 0 || fstat(fd, &st) != 0) {
    if (fd >= 0) close(fd);
    return CUDA_ERROR_INVALID_VALUE;
  }
  std::lock_guard<std::mutex> g(g_mu);
  *h = g_next_handle++;
  g_handles[*h] = VmmHandle{fd, static_cast<size_t>(st.st_size), 1, true};
  return CUDA_SUCCESS;
}
CUresult fCtxGetDevice(CUdevice* d) {
  *d = 0;
  return CUDA_SUCCESS;
}
// a "device" allocation made the way NCCL makes its buffers: create, reserve, map
CUresult vmm_style_alloc(CUdeviceptr* out, size_t bytes) {
  const size_t size = (bytes + 65535) & ~static_cast<size_t>(65535);
  CUmemGenericAllocationHandle h;
  if (fMemCreate(&h, size, nullptr, 0) != CUDA_SUCCESS) return CUDA_ERROR_OUT_OF_MEMORY;
  CUdeviceptr va = 0;
  if (fMemAddressReserve(&va, size, 0, 0, 0) != CUDA_SUCCESS || fMemMap(va, size, 0, h, 0) != CUDA_SUCCESS) return CUDA_ERROR_OUT_OF_MEMORY;
  fMemRelease(h);   // the mapping holds the allocation from here on
  *out = va;
  return CUDA_SUCCESS;
}
CUresult fNotSupported() { return CUDA_ERROR_NOT_SUPPORTED; }

struct Entry {
  const char* name;
  void* fn;
};
#define E(n, f) {n, reinterpret_cast<void*>(f)}
const Entry kTable[] = {
    E("cuInit", fInit), E("cuDeviceGetCount", fDeviceGetCount), E("cuDeviceGet", fDeviceGet),
    E("cuDeviceGetAttribute", fDeviceGetAttribute), E("cuDeviceGetP2PAttribute", fDeviceGetP2PAttribute),
    E("cuDeviceGetPCIBusId", fDeviceGetPCIBusId), E("cuDeviceGetUuid", fDeviceGetUuid),
    E("cuPointerGetAttribute", fPointerGetAttribute), E("cuMemGetAddressRange", fMemGetAddressRange),
    E("cuIpcGetMemHandle", fIpcGetMemHandle), E("cuIpcOpenMemHandle", fIpcOpenMemHandle),
    E("cuIpcCloseMemHandle", fIpcCloseMemHandle), E("cuCtxGetCurrent", fCtxGetCurrent), E("cuCtxSetCurrent", fCtxSetCurrent),
    E("cuDevicePrimaryCtxRetain", fDevicePrimaryCtxRetain), E("cuStreamCreate", fStreamCreate),
    E("cuStreamDestroy", fStreamDestroy), E("cuStreamSynchronize", fStreamSynchronize), E("cuEventCreate", fEventCreate),
    E("cuEventDestroy", fEventDestroy), E("cuEventRecord", fEventRecord), E("cuEventQuery", fEventQuery),
    E("cuMemcpyAsync", fMemcpyAsync), E("cuModuleLoadData", fModuleLoadData), E("cuModuleUnload", fModuleUnload),
    E("cuModuleGetFunction", fModuleGetFunction), E("cuLaunchKernel", fLaunchKernel), E("cuMemHostAlloc", fMemHostAlloc),
    E("cuMemFreeHost", fMemFreeHost), E("cuMemAlloc", fMemAlloc), E("cuMemFree", fMemFree), E("cuMemsetD8", fMemsetD8),
    E("cuMemCreate", fMemCreate), E("cuMemRelease", fMemRelease), E("cuMemGetAllocationGranularity", fMemGetAllocationGranularity),
    E("cuMemAddressReserve", fMemAddressReserve), E("cuMemAddressFree", fMemAddressFree), E("cuMemMap", fMemMap),
    E("cuMemUnmap", fMemUnmap), E("cuMemSetAccess", fMemSetAccess), E("cuMemExportToShareableHandle", fMemExportToShareableHandle),
    E("cuMemImportFromShareableHandle", fMemImportFromShareableHandle), E("cuMemRetainAllocationHandle", fMemRetainAllocationHandle),
    E("cuCtxGetDevice", fCtxGetDevice), E("cuMemHostRegister", fMemHostRegister), E("cuMemHostUnregister", fMemHostUnregister),
    E("cuCtxSynchronize", fCtxSynchronize), E("cuFuncSetAttribute", fFuncSetAttribute),
};

}  // namespace

extern "C" {
// The one symbol the plugin looks up with dlsym; everything else is resolved through it.
CUresult cuGetProcAddress_v2(const char* symbol, void** pfn, int, cuuint64_t, CUdriverProcAddressQueryResult* status) {
  for (const Entry& e : kTable) {
    if (!strcmp(e.name, symbol)) {
      *pfn = e.fn;
      if (status) *status = CU_GET_PROC_ADDRESS_SUCCESS;
      return CUDA_SUCCESS;
    }
  }
  *pfn = nullptr;
  if (status) *status = CU_GET_PROC_ADDRESS_SYMBOL_NOT_FOUND;
  return CUDA_ERROR_NOT_FOUND;
}
// For the tests themselves: allocate and free "device" memory without going through the table.
CUresult fake_cuda_mem_alloc(void** p, size_t bytes) {
  CUdeviceptr d = 0;
  const bool vmm = getenv("FAKE_CUDA_VMM") && atoi(getenv("FAKE_CUDA_VMM"));
  const CUresult r = vmm ? vmm_style_alloc(&d, bytes) : fMemAlloc(&d, bytes);
  *p = reinterpret_cast<void*>(d);
  return r;
}
CUresult fake_cuda_mem_free(void* p) {
  size_t vmm_size = 0;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_allocs.find(reinterpret_cast<uintptr_t>(p));
    if (it != g_allocs.end() && it->second.vmm_handle) vmm_size = it->second.size;
  }
  if (!vmm_size) return fMemFree(reinterpret_cast<CUdeviceptr>(p));
  const CUresult r = fMemUnmap(reinterpret_cast<CUdeviceptr>(p), vmm_size);
  fMemAddressFree(reinterpret_cast<CUdeviceptr>(p), vmm_size);
  return r;
}
// One address range backed by several allocations of the virtual-memory API (seg_bytes each, a
// multiple of 64 KiB), the way an application may build a large window.
CUresult fake_cuda_mem_alloc_segments(void** p, size_t seg_bytes, int nseg) {
  CUdeviceptr va = 0;
  if (seg_bytes % 65536 || nseg < 1 || fMemAddressReserve(&va, seg_bytes * nseg, 0, 0, 0) != CUDA_SUCCESS) return CUDA_ERROR_INVALID_VALUE;
  for (int i = 0; i < nseg; ++i) {
    CUmemGenericAllocationHandle h;
    if (fMemCreate(&h, seg_bytes, nullptr, 0) != CUDA_SUCCESS || fMemMap(va + i * seg_bytes, seg_bytes, 0, h, 0) != CUDA_SUCCESS)
      return CUDA_ERROR_OUT_OF_MEMORY;
    fMemRelease(h);
  }
  *p = reinterpret_cast<void*>(va);
  return CUDA_SUCCESS;
}
CUresult fake_cuda_mem_free_segments(void* p, size_t seg_bytes, int nseg) {
  for (int i = 0; i < nseg; ++i) fMemUnmap(reinterpret_cast<CUdeviceptr>(p) + i * seg_bytes, seg_bytes);
  return fMemAddressFree(reinterpret_cast<CUdeviceptr>(p), seg_bytes * nseg);
}
// How many peer allocations are mapped into this process right now (opened and not yet closed).
int fake_cuda_live_peer_mappings() {
  std::lock_guard<std::mutex> g(g_mu);
  int n = 0;
  for (const auto& [base, al] : g_allocs) n += al.opened_from_peer ? 1 : 0;
  return n;
}
// From now on the n-th asynchronous copy and every later one fails (n < 0: copies work again).
void fake_cuda_fail_memcpy_after(long n) { g_memcpy_budget.store(n); }
// The same for kernel launches.
void fake_cuda_fail_launch_after(long n) { g_launch_budget.store(n); }
// The accessible view of a "device" address (what a test uses to fill and check device buffers).
void* fake_cuda_host_view(void* p) { return dev_view(p); }
}
