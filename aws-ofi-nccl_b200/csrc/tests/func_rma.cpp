// Functional test of the RMA / GIN tables through the public ABI (dlopen + ncclRmaPlugin_v15,
// ncclGinPlugin_v13, ncclGinPlugin_v14), N processes on one host; host buffers, or with
// FUNC_NET_DEVICE=1 and the stand-in driver on the library path, device buffers:
//   * collective connect over the plugin's own ring bootstrap
//   * 64 iput + 64 iputSignal(INC) + iputSignal(ADD) to every peer; the target polls the signal
//     word while calling rmaProgress; payload verified
//   * iget from the next rank, iflush as a fence
//   * the same buffer registered twice shares one registration; dereg keeps it alive
//   * createContext of the kernel-initiated table rejects a null config and out-of-range backend
//     versions before it looks at the communicator (a dummy pointer is passed)
// usage: func_rma [plugin.so] [nranks]
#include <dlfcn.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "b200net/gin_dev_handle.h"
#include <vector>

#include "nccl_abi.h"

static int g_rank = 0, g_n = 3;
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

#include "test_buf.h"

using Clock = std::chrono::steady_clock;
static bool expired(Clock::time_point t0, int s = 30) { return Clock::now() - t0 > std::chrono::seconds(s); }

// out-of-band exchange through memory shared by all forked ranks
struct Oob {
  char handles[16][NCCL_NET_HANDLE_MAXSIZE];
  std::atomic<int> arrived[64];
  std::atomic<int> failed;
};
static Oob* oob = nullptr;
static int g_barrier_idx = 0;
static ncclRma_v15_t* g_rma = nullptr;
static void* g_progress_ctx = nullptr;
// While waiting, keep the progress engine turning (as NCCL's proxy thread would): a peer may be
// reading from this rank through the request/response path.
static int oob_barrier() {
  const int idx = g_barrier_idx++;
  oob->arrived[idx].fetch_add(1);
  const auto t0 = Clock::now();
  while (oob->arrived[idx].load() < g_n) {
    if (oob->failed.load() || expired(t0, 60)) return 1;
    if (g_rma && g_progress_ctx) g_rma->rmaProgress(g_progress_ctx);
    usleep(100);
  }
  return 0;
}

static void logger(ncclDebugLogLevel level, unsigned long, const char* file, int line, const char* fmt, ...) {
  if (level > NCCL_LOG_WARN && !getenv("FUNC_NET_VERBOSE")) return;
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  fprintf(stderr, "[rank %d] %s (%s:%d)\n", g_rank, buf, file, line);
}

static int wait_req(ncclRma_v15_t* rma, void* coll, void* ctx, void* req) {
  const auto t0 = Clock::now();
  int done = 0;
  while (!done) {
    OK(rma->test(coll, req, &done));
    OK(rma->rmaProgress(ctx));
    if (expired(t0)) FAIL("request did not complete");
  }
  return 0;
}

static int run_rank(const char* so) {
  void* h = dlopen(so, RTLD_NOW | RTLD_LOCAL);
  if (!h) FAIL("dlopen: %s", dlerror());
  for (const char* s : {"ncclGinPlugin_v11", "ncclGinPlugin_v13", "ncclGinPlugin_v14", "ncclRmaPlugin_v14", "ncclRmaPlugin_v15"})
    if (!dlsym(h, s)) FAIL("symbol %s not exported", s);
  auto* rma = static_cast<ncclRma_v15_t*>(dlsym(h, "ncclRmaPlugin_v15"));
  auto* gin14 = static_cast<ncclGin_v14_t*>(dlsym(h, "ncclGinPlugin_v14"));

  // ---- reject paths of the kernel-initiated table: nothing is initialised, the comm is a dummy
  {
    void* dummy = reinterpret_cast<void*>(0x1000);
    void* ctx = nullptr;
    ncclNetDeviceHandle_t* dh = nullptr;
    if (gin14->createContext(dummy, nullptr, &ctx, &dh) != ncclInvalidArgument) FAIL("null config accepted");
    ncclGinConfig_v14_t cfg = {4, 4, 1, 0, -1, -1, 0};
    if (gin14->createContext(dummy, &cfg, &ctx, &dh) != ncclInvalidArgument) FAIL("backend version -1 accepted");
    cfg.backendVersion = 2;
    if (gin14->createContext(dummy, &cfg, &ctx, &dh) != ncclInvalidArgument) FAIL("backend version beyond the maximum accepted");
    ncclGinProperties_v14_t gp = {true, true};
    OK(gin14->getGinProperties(&gp));
    if (gp.supportsStrongSignals || gp.supportsVASignals) FAIL("unexpected GIN properties");
  }

  void* pctx = nullptr;
  OK(rma->init(&pctx, 77, logger));
  int ndev = 0;
  OK(rma->devices(&ndev));
  ncclNetProperties_v12_t props;
  OK(rma->getProperties(0, &props));
  if (props.netDeviceType != NCCL_NET_DEVICE_GIN_PROXY) FAIL("device type %d", (int)props.netDeviceType);
  void* lcomm = nullptr;
  OK(rma->listen(pctx, 0, oob->handles[g_rank], &lcomm));
  if (oob_barrier()) FAIL("barrier");
  void* handles[16];
  for (int r = 0; r < g_n; ++r) handles[r] = oob->handles[r];
  void* coll = nullptr;
  OK(rma->connect(pctx, handles, g_n, g_rank, lcomm, &coll));
  ncclRmaConfig_t cfg = {1, -1, 0};
  void* ctx = nullptr;
  OK(rma->createContext(coll, &cfg, &ctx));
  g_rma = rma;
  g_progress_ctx = ctx;

  // ---- buffers: data window (slot per source rank), signal words, source payload
  const size_t SLOT = 4096;
  TestBuf window_b, src_b, got_b, signals_b;
  // FUNC_RMA_HOST_TARGETS=1 keeps the put targets (window, signals) in host memory while the
  // sources stay on the device; FUNC_RMA_HOST_SOURCES=1 the other way round (=2: the buffer that
  // iget fills stays on the device, so a read of host memory lands in device memory)
  const bool host_targets = getenv("FUNC_RMA_HOST_TARGETS") && atoi(getenv("FUNC_RMA_HOST_TARGETS"));
  const bool host_sources = getenv("FUNC_RMA_HOST_SOURCES") && atoi(getenv("FUNC_RMA_HOST_SOURCES"));
  // FUNC_RMA_MULTISEG=1 (stand-in driver only): the signal words live in one address range backed by
  // two separate allocations, and ranks signal into different ones
  const size_t SEG = 65536;
  const bool multiseg = device_mode_kind() == BUF_VIEW && getenv("FUNC_RMA_MULTISEG") && atoi(getenv("FUNC_RMA_MULTISEG"));
  using SegAlloc = int (*)(void**, size_t, int);
  using SegFree = int (*)(void*, size_t, int);
  SegAlloc seg_alloc = nullptr;
  SegFree seg_free = nullptr;
  if (multiseg) {
    void* drv = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    seg_alloc = drv ? reinterpret_cast<SegAlloc>(dlsym(drv, "fake_cuda_mem_alloc_segments")) : nullptr;
    seg_free = drv ? reinterpret_cast<SegFree>(dlsym(drv, "fake_cuda_mem_free_segments")) : nullptr;
    if (!seg_alloc || !seg_free) FAIL("the stand-in driver offers no segmented allocation");
  }
  auto sig_off = [&](int r) -> uint64_t { return multiseg ? (r % 2) * SEG + static_cast<uint64_t>(r) * 8 : static_cast<uint64_t>(r) * 8; };
  const size_t sig_bytes = multiseg ? 2 * SEG : 16 * 8;
  if (buf_alloc(&window_b, SLOT * g_n, !host_targets) || buf_alloc(&src_b, SLOT, !host_sources) ||
      buf_alloc(&got_b, SLOT, !host_sources || atoi(getenv("FUNC_RMA_HOST_SOURCES")) == 2))
    FAIL("buffer allocation failed");
  if (multiseg) {
    void* p = nullptr;
    if (seg_alloc(&p, SEG, 2) != 0) FAIL("segmented allocation failed");
    signals_b.p = static_cast<uint8_t*>(p);
    signals_b.h = nullptr;   // two separate views: looked up per word below
    signals_b.n = sig_bytes;
    signals_b.dev = true;
  } else if (buf_alloc(&signals_b, sig_bytes, !host_targets)) {
    FAIL("buffer allocation failed");
  }
  auto sig_word = [&](int r) -> uint64_t* {
    return multiseg ? static_cast<uint64_t*>(g_dev_view(signals_b.data() + sig_off(r)))
                    : reinterpret_cast<uint64_t*>(signals_b.host() + sig_off(r));
  };
  // window / src / got / signals: where this test reads and writes; the *_b.data() addresses are
  // what the plugin gets (the same in host mode, inaccessible to host code in device mode)
  uint8_t *window = window_b.host(), *src = src_b.host(), *got = got_b.host();
  memset(window, 0, SLOT * g_n);
  memset(got, 0, SLOT);
  for (int r = 0; r < 16; ++r) *sig_word(r) = 0;
  for (size_t i = 0; i < SLOT; ++i) src[i] = static_cast<uint8_t>(i * 7 + g_rank);
  if (window_b.to_device() || src_b.to_device() || got_b.to_device() || (!multiseg && signals_b.to_device())) FAIL("copy to the device failed");
  void *win_mh, *src_mh, *sig_mh, *got_mh;
  OK(rma->regMrSym(coll, window_b.data(), SLOT * g_n, buf_type(window_b), 0, &win_mh));
  OK(rma->regMrSym(coll, src_b.data(), SLOT, buf_type(src_b), 0, &src_mh));
  OK(rma->regMrSym(coll, signals_b.data(), sig_bytes, buf_type(signals_b), NCCL_NET_MR_FLAG_SIGNAL_NEVER_RESET, &sig_mh));
  OK(rma->regMrSym(coll, got_b.data(), SLOT, buf_type(got_b), 0, &got_mh));

  // duplicate registration: same handle, and it survives one dereg
  void* dup = nullptr;
  OK(rma->regMrSym(coll, window_b.data(), SLOT * g_n, buf_type(window_b), 0, &dup));
  if (dup != win_mh) FAIL("a second registration of the same buffer got a different handle");
  OK(rma->deregMrSym(coll, dup));

  // ---- puts: 64 plain + 64 with INC to every peer, then one ADD of 1000
  for (int p = 0; p < g_n; ++p) {
    if (p == g_rank) continue;
    for (int i = 0; i < 128; ++i) {
      void* req = nullptr;
      const auto t0 = Clock::now();
      while (!req) {
        if (i % 2 == 0)
          OK(rma->iput(ctx, 0, (i % 16) * 256, src_mh, 256, g_rank * SLOT + (i % 16) * 256, win_mh, p, 0, &req));
        else
          OK(rma->iputSignal(ctx, 0, (i % 16) * 256, src_mh, 256, g_rank * SLOT + (i % 16) * 256, win_mh, p, sig_off(g_rank),
                             sig_mh, 1, NCCL_NET_SIGNAL_OP_INC, false, 0, &req));
        OK(rma->rmaProgress(ctx));
        if (expired(t0)) FAIL("iput kept returning no request");
      }
      if (wait_req(rma, coll, ctx, req)) return 1;
    }
    void* req = nullptr;
    OK(rma->iputSignal(ctx, 0, 0, src_mh, 0, 0, win_mh, p, sig_off(g_rank), sig_mh, 1000, NCCL_NET_SIGNAL_OP_ADD, true,
                       ncclRmaOptFlagsAggregateRequests, &req));
    if (!req) FAIL("signal-only put returned no request");
    if (wait_req(rma, coll, ctx, req)) return 1;
  }
  // ---- targets: wait for 64 + 1000 from every peer, then check the payload
  {
    const auto t0 = Clock::now();
    for (;;) {
      OK(rma->rmaProgress(ctx));
      if (!multiseg && signals_b.from_device()) FAIL("copy from the device failed");
      bool all = true;
      for (int p = 0; p < g_n; ++p)
        if (p != g_rank && __atomic_load_n(sig_word(p), __ATOMIC_ACQUIRE) != 1064) all = false;
      if (all) break;
      if (expired(t0)) FAIL("signals did not reach 1064: %llu %llu %llu", (unsigned long long)*sig_word(0),
                            (unsigned long long)*sig_word(1), (unsigned long long)*sig_word(2));
    }
    if (window_b.from_device()) FAIL("copy from the device failed");
    for (int p = 0; p < g_n; ++p) {
      if (p == g_rank) continue;
      for (size_t i = 0; i < SLOT; ++i)
        if (window[p * SLOT + i] != static_cast<uint8_t>(i * 7 + p)) FAIL("payload from rank %d differs at byte %zu", p, i);
    }
  }
  if (oob_barrier()) FAIL("barrier");
  // ---- get from the next rank's source buffer, fenced by a flush
  {
    const int peer = (g_rank + 1) % g_n;
    void* req = nullptr;
    OK(rma->iget(ctx, 0, 0, src_mh, SLOT, 0, got_mh, peer, 0, &req));
    if (!req) FAIL("iget returned no request");
    if (wait_req(rma, coll, ctx, req)) return 1;
    OK(rma->iflush(ctx, 0, got_mh, peer, &req));
    if (req && wait_req(rma, coll, ctx, req)) return 1;
    if (got_b.from_device()) FAIL("copy from the device failed");
    for (size_t i = 0; i < SLOT; ++i)
      if (got[i] != static_cast<uint8_t>(i * 7 + peer)) FAIL("iget payload differs at byte %zu", i);
  }
  // ---- kernel-initiated context (device buffers only): every rank allocates a pad of signal and
  // counter words on its device, the pads are mapped into every peer, and the device-visible
  // handle block lists {rank, nranks, signals, counters, pad address per rank}
  if (device_mode_kind() == BUF_VIEW) {   // reads the pads through the stand-in's host view
    ncclGinConfig_v14_t kcfg = {3 + g_rank, 2, 1, 0, -1, 0, 0};   // ranks ask for different counts
    void* kctx = nullptr;
    ncclNetDeviceHandle_t* dh = nullptr;
    // without legacy IPC (handles cannot be made, or cannot be opened) the pads cannot be shared:
    // the call must fail on every rank and leave nothing behind
    const bool no_ipc = (getenv("FAKE_CUDA_FAIL_IPC_GET") && atoi(getenv("FAKE_CUDA_FAIL_IPC_GET"))) ||
                        (getenv("FAKE_CUDA_FAIL_IPC_OPEN") && atoi(getenv("FAKE_CUDA_FAIL_IPC_OPEN")));
    if (no_ipc) {
      if (gin14->createContext(coll, &kcfg, &kctx, &dh) == ncclSuccess) FAIL("a context without shared pads was handed out");
      if (oob_barrier()) FAIL("barrier");
    } else {
    OK(gin14->createContext(coll, &kcfg, &kctx, &dh));
    if (!dh || dh->netDeviceType != NCCL_NET_DEVICE_GIN_GDAKI || dh->needsProxyProgress) FAIL("unexpected device handle");
    if (dh->size != sizeof(b200::GinDevHandle)) FAIL("handle of %zu bytes", (size_t)dh->size);
    const auto* hd = static_cast<const b200::GinDevHandle*>(g_dev_view(dh->handle));
    if (hd->rank != g_rank || hd->nranks != g_n || !hd->status || hd->wait_limit_ns == 0)
      FAIL("handle says rank %d of %d, status %p, wait limit %llu", hd->rank, hd->nranks, (void*)hd->status,
           (unsigned long long)hd->wait_limit_ns);
    if (reinterpret_cast<uint8_t*>(hd->status) != hd->pad[g_rank] + b200::GIN_PAD_STATUS_OFF) FAIL("status word is not inside the own pad");
    // each rank leaves its mark in signal word [rank] of every pad through the mapping it was given
    for (int r = 0; r < g_n; ++r) {
      if (!hd->pad[r]) FAIL("pad of rank %d is not mapped", r);
      auto* sig = reinterpret_cast<uint64_t*>(static_cast<uint8_t*>(g_dev_view(hd->pad[r])) + b200::GIN_PAD_SIGNAL_OFF);
      __atomic_store_n(&sig[g_rank], 0xAB00u + g_rank, __ATOMIC_RELEASE);
    }
    if (oob_barrier()) FAIL("barrier");
    const auto* mine = reinterpret_cast<const uint64_t*>(static_cast<const uint8_t*>(g_dev_view(hd->pad[g_rank])) + b200::GIN_PAD_SIGNAL_OFF);
    for (int r = 0; r < g_n; ++r)
      if (__atomic_load_n(&mine[r], __ATOMIC_ACQUIRE) != 0xAB00u + r) FAIL("pad word %d holds %llx", r, (unsigned long long)mine[r]);
    if (oob_barrier()) FAIL("barrier");
    OK(gin14->destroyContext(kctx));
    }
  }
  bool err = true;
  OK(rma->queryLastError(ctx, &err));
  if (err) FAIL("queryLastError reports an error");
  if (oob_barrier()) FAIL("barrier");
  g_progress_ctx = nullptr;
  OK(rma->deregMrSym(coll, got_mh));
  OK(rma->deregMrSym(coll, sig_mh));
  OK(rma->deregMrSym(coll, src_mh));
  OK(rma->deregMrSym(coll, win_mh));
  buf_free(&window_b);
  buf_free(&src_b);
  buf_free(&got_b);
  if (multiseg) seg_free(signals_b.data(), SEG, 2);
  else buf_free(&signals_b);
  OK(rma->destroyContext(ctx));
  OK(rma->closeColl(coll));
  OK(rma->closeListen(lcomm));
  OK(rma->finalize(pctx));
  return 0;
}

int main(int argc, char** argv) {
  const char* so = argc > 1 ? argv[1] : "./libnccl-net-ofi-b200.so";
  g_n = argc > 2 ? atoi(argv[2]) : 3;
  if (g_n < 1 || g_n > 16) return 2;
  oob = static_cast<Oob*>(mmap(nullptr, sizeof(Oob), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
  if (oob == MAP_FAILED) return 2;
  memset(static_cast<void*>(oob), 0, sizeof(Oob));
  std::vector<pid_t> kids;
  for (int r = 1; r < g_n; ++r) {
    const pid_t pid = fork();
    if (pid < 0) return 2;
    if (pid == 0) {
      g_rank = r;
      const int rc = run_rank(so);
      if (rc) oob->failed.store(1);
      _exit(rc);
    }
    kids.push_back(pid);
  }
  g_rank = 0;
  int rc = run_rank(so);
  if (rc) oob->failed.store(1);
  for (pid_t k : kids) {
    int st = 0;
    waitpid(k, &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st)) rc = 1;
  }
  if (rc) {
    fprintf(stderr, "FAILED\n");
    return 1;
  }
  printf("ok\n");
  return 0;
}
