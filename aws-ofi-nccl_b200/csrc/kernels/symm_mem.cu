// Symmetric memory over CUDA VMM: every rank allocates one physical chunk, exports it as a POSIX
// file descriptor, passes the descriptor to its peers over an abstract unix socket (SCM_RIGHTS),
// and maps all chunks into one contiguous virtual range (peer i at base + i * chunk). An optional
// NVSwitch multicast object is bound over the same chunks for multimem loads/stores.
//
// This is the "memory registration + address exchange" of the NVLink fabric: what fi_mr_reg, rkeys
// and the address vector are to the reference's libfabric transport
// (reference: src/nccl_ofi_cuda.cpp VMM allocation :481-568, src/rdma/gin/nccl_ofi_gin.cpp
// symmetric registration :317-425).
#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <poll.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <mutex>
#include <thread>
#include <vector>

#include "host_util.h"

namespace b200 {

struct Drv {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                         unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                               unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  bool ok = false;
};

template <typename F>
static bool resolve(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    return false;
  fn = reinterpret_cast<F>(p);
  return true;
}

static Drv& drv() {
  static Drv d;
  static std::once_flag once;
  std::call_once(once, [] {
    bool ok = true;
    ok &= resolve(d.MemCreate, "cuMemCreate");
    ok &= resolve(d.MemRelease, "cuMemRelease");
    ok &= resolve(d.MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    ok &= resolve(d.MemExportToShareableHandle, "cuMemExportToShareableHandle");
    ok &= resolve(d.MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    ok &= resolve(d.MemAddressReserve, "cuMemAddressReserve");
    ok &= resolve(d.MemAddressFree, "cuMemAddressFree");
    ok &= resolve(d.MemMap, "cuMemMap");
    ok &= resolve(d.MemUnmap, "cuMemUnmap");
    ok &= resolve(d.MemSetAccess, "cuMemSetAccess");
    ok &= resolve(d.MulticastCreate, "cuMulticastCreate");
    ok &= resolve(d.MulticastAddDevice, "cuMulticastAddDevice");
    ok &= resolve(d.MulticastBindMem, "cuMulticastBindMem");
    ok &= resolve(d.MulticastUnbind, "cuMulticastUnbind");
    ok &= resolve(d.MulticastGetGranularity, "cuMulticastGetGranularity");
    ok &= resolve(d.DeviceGetAttribute, "cuDeviceGetAttribute");
    d.ok = ok;
  });
  return d;
}

#define DRV_OK(expr)                                                                             \
  do {                                                                                           \
    CUresult _r = (expr);                                                                        \
    if (_r != CUDA_SUCCESS) {                                                                    \
      fprintf(stderr, "[b200ops] %s:%d %s -> CUresult %d\n", __FILE__, __LINE__, #expr, (int)_r); \
      return 20000 + static_cast<int>(_r);                                                       \
    }                                                                                            \
  } while (0)

struct SymmAlloc {
  int device = 0;
  int world = 0, rank = 0;
  size_t chunk = 0;  // bytes per rank (granularity aligned)
  CUmemGenericAllocationHandle local = 0;
  std::vector<CUmemGenericAllocationHandle> peers;  // imported handles (own slot = local)
  CUdeviceptr base = 0;                             // world * chunk bytes of VA
  CUmemGenericAllocationHandle mc = 0;
  CUdeviceptr mc_ptr = 0;
  bool mc_bound = false;
};

static std::mutex g_mu;
static std::vector<SymmAlloc*> g_allocs;

static SymmAlloc* get_alloc(int id) {
  std::lock_guard<std::mutex> g(g_mu);
  if (id < 0 || id >= static_cast<int>(g_allocs.size())) return nullptr;
  return g_allocs[id];
}

static CUmemAllocationProp local_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

// ---------------------------------------------------------------- fd passing over abstract unix sockets
static void make_addr(const char* name, sockaddr_un* addr, socklen_t* len) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  const size_t n = strnlen(name, sizeof(addr->sun_path) - 2);
  memcpy(addr->sun_path + 1, name, n);  // leading NUL = abstract namespace (no filesystem entry)
  *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

static int send_fd(int sock, int fd) {
  char data = 'F';
  iovec iov{&data, 1};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, 0) == 1 ? 0 : -errno;
}

static int recv_fd(int sock) {
  char data = 0;
  iovec iov{&data, 1};
  char ctrl[CMSG_SPACE(sizeof(int))];
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &msg, 0) != 1) return -1;
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return -1;
  int fd = -1;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  return fd;
}

struct FdServer {
  int listen_fd = -1;
  std::vector<int> fds;
  int remaining = 0;
  std::thread th;
};
static std::vector<FdServer*> g_servers;

static void serve(FdServer* s, int timeout_ms) {
  while (s->remaining > 0) {
    pollfd p{s->listen_fd, POLLIN, 0};
    if (poll(&p, 1, timeout_ms) <= 0) break;  // nobody came: give up instead of blocking forever
    int c = accept(s->listen_fd, nullptr, nullptr);
    if (c < 0) continue;
    int idx = -1;
    if (read(c, &idx, sizeof(idx)) == sizeof(idx) && idx >= 0 && idx < static_cast<int>(s->fds.size()))
      send_fd(c, s->fds[idx]);
    close(c);
    --s->remaining;
  }
  close(s->listen_fd);
  s->listen_fd = -1;
}

}  // namespace b200

extern "C" {
using namespace b200;

// 1 if the current device supports NVSwitch multicast objects, 0 if not, <0 on error.
int b200_symm_multicast_supported(int device) {
  ensure_context();
  Drv& d = drv();
  if (!d.ok) return -1;
  int v = 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return -1;
  return v;
}

// Allocate this rank's chunk. `bytes` is rounded up to the allocation (and multicast) granularity;
// the rounded size is returned through chunk_out and must be identical on all ranks.
int b200_symm_alloc(size_t bytes, int device, int world, int rank, int want_multicast, int* id_out,
                    size_t* chunk_out) {
  ensure_context();
  Drv& d = drv();
  if (!d.ok) return B200_ERR_NO_DRIVER;
  CUmemAllocationProp prop = local_prop(device);
  size_t gran = 0;
  DRV_OK(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (want_multicast) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(world);
    mp.size = bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  const size_t chunk = (bytes + gran - 1) / gran * gran;
  auto* a = new SymmAlloc();
  a->device = device;
  a->world = world;
  a->rank = rank;
  a->chunk = chunk;
  a->peers.assign(world, 0);
  CUresult r = d.MemCreate(&a->local, chunk, &prop, 0);
  if (r != CUDA_SUCCESS) {
    delete a;
    fprintf(stderr, "[b200ops] cuMemCreate(%zu) failed: %d\n", chunk, (int)r);
    return 20000 + static_cast<int>(r);
  }
  a->peers[rank] = a->local;
  std::lock_guard<std::mutex> g(g_mu);
  g_allocs.push_back(a);
  *id_out = static_cast<int>(g_allocs.size()) - 1;
  *chunk_out = chunk;
  return 0;
}

// Export the local chunk (which = 0) or the multicast object (which = 1) as a file descriptor.
int b200_symm_export_fd(int id, int which, int* fd_out) {
  SymmAlloc* a = get_alloc(id);
  if (!a) return B200_ERR_BAD_ARG;
  int fd = -1;
  DRV_OK(drv().MemExportToShareableHandle(&fd, which ? a->mc : a->local, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd_out = fd;
  return 0;
}

// Serve `nclients` requests for the given descriptors on an abstract unix socket, on a helper
// thread that exits after the last request or after timeout_ms without a connection.
int b200_fd_server_start(const char* name, const int* fds, int nfds, int nclients, int timeout_ms, int* server_out) {
  auto* s = new FdServer();
  s->listen_fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s->listen_fd < 0) return -errno;
  sockaddr_un addr;
  socklen_t len;
  make_addr(name, &addr, &len);
  if (bind(s->listen_fd, reinterpret_cast<sockaddr*>(&addr), len) != 0 || listen(s->listen_fd, 64) != 0) {
    const int e = errno;
    close(s->listen_fd);
    delete s;
    return -e;
  }
  s->fds.assign(fds, fds + nfds);
  s->remaining = nclients;
  s->th = std::thread(serve, s, timeout_ms);
  std::lock_guard<std::mutex> g(g_mu);
  g_servers.push_back(s);
  *server_out = static_cast<int>(g_servers.size()) - 1;
  return 0;
}

int b200_fd_server_join(int server) {
  FdServer* s;
  {
    std::lock_guard<std::mutex> g(g_mu);
    if (server < 0 || server >= static_cast<int>(g_servers.size()) || !g_servers[server]) return B200_ERR_BAD_ARG;
    s = g_servers[server];
    g_servers[server] = nullptr;
  }
  if (s->th.joinable()) s->th.join();
  const int left = s->remaining;
  delete s;
  return left;  // 0 when every expected client was served
}

// Ask the server at `name` for descriptor `index`. Retries the connect until timeout_ms.
int b200_fd_fetch(const char* name, int index, int timeout_ms, int* fd_out) {
  sockaddr_un addr;
  socklen_t len;
  make_addr(name, &addr, &len);
  for (int waited = 0;; waited += 10) {
    int c = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (c < 0) return -errno;
    if (connect(c, reinterpret_cast<sockaddr*>(&addr), len) == 0) {
      int rc = 0;
      if (write(c, &index, sizeof(index)) != sizeof(index)) rc = -EIO;
      const int fd = rc ? -1 : recv_fd(c);
      close(c);
      if (fd < 0) return -EIO;
      *fd_out = fd;
      return 0;
    }
    close(c);
    if (waited >= timeout_ms) return -ETIMEDOUT;
    usleep(10000);
  }
}

// Import the peers' chunks (fds[i] for rank i, ignored for the own rank; descriptors are closed)
// and map everything: peer i at base + i * chunk, read/write for this device.
int b200_symm_map(int id, const int* fds, void** base_out) {
  ensure_context();
  SymmAlloc* a = get_alloc(id);
  if (!a) return B200_ERR_BAD_ARG;
  Drv& d = drv();
  for (int i = 0; i < a->world; ++i) {
    if (i == a->rank) continue;
    DRV_OK(d.MemImportFromShareableHandle(&a->peers[i], reinterpret_cast<void*>(static_cast<intptr_t>(fds[i])),
                                          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    close(fds[i]);
  }
  DRV_OK(d.MemAddressReserve(&a->base, a->chunk * a->world, 0, 0, 0));
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = a->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int i = 0; i < a->world; ++i) {
    DRV_OK(d.MemMap(a->base + i * a->chunk, a->chunk, 0, a->peers[i], 0));
    DRV_OK(d.MemSetAccess(a->base + i * a->chunk, a->chunk, &acc, 1));
  }
  *base_out = reinterpret_cast<void*>(a->base);
  return 0;
}

// Multicast, step 1 (rank 0 only): create the object sized for one chunk.
int b200_symm_mc_create(int id) {
  ensure_context();
  SymmAlloc* a = get_alloc(id);
  if (!a) return B200_ERR_BAD_ARG;
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = static_cast<unsigned>(a->world);
  mp.size = a->chunk;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  DRV_OK(drv().MulticastCreate(&a->mc, &mp));
  return 0;
}
// step 1' (other ranks): import rank 0's object.
int b200_symm_mc_import(int id, int fd) {
  ensure_context();
  SymmAlloc* a = get_alloc(id);
  if (!a) return B200_ERR_BAD_ARG;
  DRV_OK(drv().MemImportFromShareableHandle(&a->mc, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  close(fd);
  return 0;
}
// step 2 (all ranks, then barrier): join the team.
int b200_symm_mc_add_device(int id) {
  ensure_context();
  SymmAlloc* a = get_alloc(id);
  if (!a || !a->mc) return B200_ERR_BAD_ARG;
  DRV_OK(drv().MulticastAddDevice(a->mc, a->device));
  return 0;
}
// step 3 (all ranks, after every rank added its device): bind the local chunk and map the object.
int b200_symm_mc_bind_map(int id, void** mc_ptr_out) {
  ensure_context();
  SymmAlloc* a = get_alloc(id);
  if (!a || !a->mc) return B200_ERR_BAD_ARG;
  Drv& d = drv();
  DRV_OK(d.MulticastBindMem(a->mc, 0, a->local, 0, a->chunk, 0));
  a->mc_bound = true;
  DRV_OK(d.MemAddressReserve(&a->mc_ptr, a->chunk, 0, 0, 0));
  DRV_OK(d.MemMap(a->mc_ptr, a->chunk, 0, a->mc, 0));
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = a->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  DRV_OK(d.MemSetAccess(a->mc_ptr, a->chunk, &acc, 1));
  *mc_ptr_out = reinterpret_cast<void*>(a->mc_ptr);
  return 0;
}

// Unmap and release everything of this allocation. Call on every rank, after a barrier, with no
// kernel in flight that touches the memory.
int b200_symm_free(int id) {
  ensure_context();
  SymmAlloc* a = get_alloc(id);
  if (!a) return B200_ERR_BAD_ARG;
  Drv& d = drv();
  if (a->mc_ptr) {
    d.MemUnmap(a->mc_ptr, a->chunk);
    d.MemAddressFree(a->mc_ptr, a->chunk);
  }
  if (a->mc) {
    if (a->mc_bound) d.MulticastUnbind(a->mc, a->device, 0, a->chunk);
    d.MemRelease(a->mc);
  }
  if (a->base) {
    for (int i = 0; i < a->world; ++i) d.MemUnmap(a->base + i * a->chunk, a->chunk);
    d.MemAddressFree(a->base, a->chunk * a->world);
  }
  for (int i = 0; i < a->world; ++i)
    if (a->peers[i]) d.MemRelease(a->peers[i]);
  {
    std::lock_guard<std::mutex> g(g_mu);
    g_allocs[id] = nullptr;
  }
  delete a;
  return 0;
}

}  // extern "C"
