// Kernel-initiated GIN end to end on real GPUs: two processes load the plugin, connect through the
// exported ncclGinPlugin_v14 table, register a device window (regMrSym hands back the device
// address of its GinDevWindow), create a kernel-initiated context (createContext hands back the
// device address of its GinDevHandle) and then a <<<1,1>>> kernel of one rank puts 64 bytes into
// the other rank's window and raises a signal there, all through the handles the PLUGIN built and
// the device API of kernels/gin_device.cuh. The target's kernel waits for the signal with a bound
// and returns a status; the host checks the payload, the signal value and the status word.
// (reference: tests/functional/gin_put_gdaki_gpu.cu:45-92, gin_signal_gdaki_gpu.cu:41-92.)
//
// The two kernels never wait for each other at the same time: the put kernel has finished (host
// barrier) before the wait kernel starts, so the test is also safe when both ranks share one GPU.
// Exit status 0 = pass, 77 = no GPU.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "gin_device.cuh"
#include "nccl_abi.h"

using namespace b200;

static int g_rank = 0;
#define FAIL(...)                                                     \
  do {                                                                \
    fprintf(stderr, "[rank %d] %s:%d: ", g_rank, __FILE__, __LINE__); \
    fprintf(stderr, __VA_ARGS__);                                     \
    fprintf(stderr, "\n");                                            \
    return 1;                                                         \
  } while (0)
#define OK(call)                                                   \
  do {                                                             \
    ncclResult_t _r = (call);                                      \
    if (_r != ncclSuccess) FAIL("%s returned %d", #call, (int)_r); \
  } while (0)
#define CU(call)                                                                      \
  do {                                                                                \
    cudaError_t _e = (call);                                                          \
    if (_e != cudaSuccess) FAIL("%s: %s", #call, cudaGetErrorString(_e));             \
  } while (0)

__global__ void put_signal_kernel(const GinDevHandle* h, const GinDevWindow* w, int peer, size_t dst_off, const uint8_t* src,
                                  size_t bytes, int sig, int* result) {
  const bool ok = gin_put_window(*h, *w, peer, dst_off, src, bytes, 0, 1);
  if (ok) gin_signal(*h, peer, sig, 1, GIN_SIGNAL_INC);   // release-ordered behind the payload
  gin_counter_add(*h, 0, 1);                              // local completion counter
  *result = ok ? 1 : -1;
}

__global__ void wait_signal_kernel(const GinDevHandle* h, int sig, unsigned long long target, int* result,
                                   unsigned long long* seen) {
  const bool ok = gin_wait_signal(*h, sig, target);   // bounded: gives up after the handle's wait limit
  *seen = gin_read_signal(*h, sig);
  *result = ok ? 1 : -1;
}

static void logger(ncclDebugLogLevel level, unsigned long, const char*, int, const char* fmt, ...) {
  if (level > NCCL_LOG_WARN && !getenv("GIN_TEST_VERBOSE")) return;
  va_list ap;
  va_start(ap, fmt);
  fprintf(stderr, "[rank %d] ", g_rank);
  vfprintf(stderr, fmt, ap);
  fprintf(stderr, "\n");
  va_end(ap);
}

static int xchg(int sock, const void* mine, void* theirs, size_t n) {
  if (write(sock, mine, n) != (ssize_t)n) return 1;
  size_t got = 0;
  while (got < n) {
    const ssize_t r = read(sock, static_cast<char*>(theirs) + got, n - got);
    if (r <= 0) return 1;
    got += static_cast<size_t>(r);
  }
  return 0;
}
static int barrier(int sock) {
  char a = 1, b = 0;
  return xchg(sock, &a, &b, 1);
}

static int run_rank(const char* so, int sock) {
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < 1) return 77;
  CU(cudaSetDevice(g_rank % ndev));
  CU(cudaFree(nullptr));
  setenv("B200NET_DEVICE_WAIT_LIMIT_MS", "1000", 0);   // every device wait of this test gives up after a second
  void* lib = dlopen(so, RTLD_NOW | RTLD_LOCAL);
  if (!lib) FAIL("dlopen(%s): %s", so, dlerror());
  auto* gin = static_cast<ncclGin_v14_t*>(dlsym(lib, "ncclGinPlugin_v14"));
  if (!gin) FAIL("ncclGinPlugin_v14 not exported");
  void* pctx = nullptr;
  OK(gin->init(&pctx, 0x6147, logger));
  ncclGinProperties_v14_t gp;
  memset(&gp, 0, sizeof(gp));
  OK(gin->getGinProperties(&gp));
  char mine[NCCL_NET_HANDLE_MAXSIZE] = {0}, theirs[NCCL_NET_HANDLE_MAXSIZE] = {0};
  void *lcomm = nullptr, *coll = nullptr;
  OK(gin->listen(pctx, g_rank % ndev, mine, &lcomm));
  if (xchg(sock, mine, theirs, sizeof(mine))) FAIL("handle exchange");
  void* handles[2];
  handles[g_rank] = mine;
  handles[1 - g_rank] = theirs;
  OK(gin->connect(pctx, handles, 2, g_rank, lcomm, &coll));

  // a device window and its registration: the plugin maps the peer's window and describes both to the GPU
  const size_t WIN = 64 << 10;
  uint8_t *window = nullptr, *src = nullptr;
  CU(cudaMalloc(&window, WIN));
  CU(cudaMemset(window, 0xEE, WIN));
  CU(cudaMalloc(&src, 256));
  std::vector<uint8_t> pattern(256);
  for (size_t i = 0; i < pattern.size(); ++i) pattern[i] = static_cast<uint8_t>(17 * i + 3 + 100 * g_rank);
  CU(cudaMemcpy(src, pattern.data(), pattern.size(), cudaMemcpyHostToDevice));
  CU(cudaDeviceSynchronize());
  void *mh = nullptr, *dev_window = nullptr;
  OK(gin->regMrSym(coll, window, WIN, NCCL_PTR_CUDA, 0, &mh, &dev_window));
  if (!dev_window) FAIL("regMrSym returned no device window");
  ncclGinConfig_v14_t cfg = {8, 2, 1, 0, -1, 0, 0};
  void* kctx = nullptr;
  ncclNetDeviceHandle_t* dh = nullptr;
  OK(gin->createContext(coll, &cfg, &kctx, &dh));
  if (!dh || !dh->handle || dh->size != sizeof(GinDevHandle) || dh->needsProxyProgress) FAIL("unexpected device handle");
  const auto* h = static_cast<const GinDevHandle*>(dh->handle);
  const auto* w = static_cast<const GinDevWindow*>(dev_window);

  int* result = nullptr;
  unsigned long long* seen = nullptr;
  CU(cudaMallocHost(&result, sizeof(int)));
  CU(cudaMallocHost(&seen, sizeof(*seen)));
  const int SIG = 5;
  const size_t OFF = 4096 + 64 * g_rank;
  for (int dir = 0; dir < 2; ++dir) {   // rank `dir` puts, the other waits
    const int sender = dir, target = 1 - dir;
    if (barrier(sock)) FAIL("barrier");
    if (g_rank == sender) {
      *result = 0;
      put_signal_kernel<<<1, 1>>>(h, w, target, 4096 + 64 * sender, src, 64, SIG, result);
      CU(cudaGetLastError());
      CU(cudaDeviceSynchronize());
      if (*result != 1) FAIL("the put kernel reported %d", *result);
    }
    if (barrier(sock)) FAIL("barrier");   // the put kernel has finished before the wait kernel starts
    if (g_rank == target) {
      *result = 0;
      *seen = 0;
      wait_signal_kernel<<<1, 1>>>(h, SIG, 1, result, seen);
      CU(cudaGetLastError());
      CU(cudaDeviceSynchronize());
      if (*result != 1) FAIL("the signal did not arrive within the wait limit (saw %llu)", *seen);
      if (*seen != 1) FAIL("signal value %llu, expected 1", *seen);
      std::vector<uint8_t> got(WIN);
      CU(cudaMemcpy(got.data(), window, WIN, cudaMemcpyDeviceToHost));
      const size_t at = 4096 + 64 * sender;
      for (size_t i = 0; i < 64; ++i)
        if (got[at + i] != static_cast<uint8_t>(17 * i + 3 + 100 * sender)) FAIL("payload byte %zu is %02x", i, got[at + i]);
      if (got[at - 1] != 0xEE || got[at + 64] != 0xEE) FAIL("the put wrote outside its 64 bytes");
    }
  }
  (void)OFF;
  // a wait for a signal nobody raises gives up after the limit and records it in the status word
  if (barrier(sock)) FAIL("barrier");
  *result = 0;
  wait_signal_kernel<<<1, 1>>>(h, SIG + 1, 1, result, seen);
  CU(cudaDeviceSynchronize());
  if (*result != -1) FAIL("a wait on a silent signal returned %d", *result);
  GinDevHandle host_h;
  CU(cudaMemcpy(&host_h, h, sizeof(host_h), cudaMemcpyDeviceToHost));
  int status = 0;
  CU(cudaMemcpy(&status, host_h.status, sizeof(int), cudaMemcpyDeviceToHost));
  if (status == 0) FAIL("the status word stayed clear after a wait ran out");
  bool err = false;
  OK(gin->queryLastError(kctx, &err));
  if (barrier(sock)) FAIL("barrier");
  OK(gin->destroyContext(kctx));
  OK(gin->deregMrSym(coll, mh));
  OK(gin->closeColl(coll));
  OK(gin->closeListen(lcomm));
  OK(gin->finalize(pctx));
  cudaFree(window);
  cudaFree(src);
  fprintf(stderr, "[rank %d] kernel-initiated put + signal through plugin-built handles: ok\n", g_rank);
  return 0;
}

int main(int argc, char** argv) {
  const char* so = argc > 1 ? argv[1] : "./libnccl-net-ofi-b200.so";
  int sv[2];
  if (socketpair(AF_UNIX, SOCK_STREAM, 0, sv) != 0) return 2;
  const pid_t pid = fork();   // before any CUDA call
  if (pid < 0) return 2;
  if (pid == 0) {
    close(sv[0]);
    g_rank = 1;
    _exit(run_rank(so, sv[1]));
  }
  close(sv[1]);
  g_rank = 0;
  const int rc0 = run_rank(so, sv[0]);
  close(sv[0]);
  int status = 0;
  waitpid(pid, &status, 0);
  const int rc1 = WIFEXITED(status) ? WEXITSTATUS(status) : 3;
  if (rc0 == 77 && rc1 == 77) return 77;
  if (rc0 || rc1) {
    fprintf(stderr, "FAILED: rank0=%d rank1=%d\n", rc0, rc1);
    return 1;
  }
  printf("ok\n");
  return 0;
}
