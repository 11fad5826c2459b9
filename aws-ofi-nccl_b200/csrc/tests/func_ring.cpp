// Ring of N processes over the net plugin's public ABI (dlopen + ncclNetPlugin_v11): every rank
// listens, connects to rank+1 and accepts from rank-1; then, per round, 32 sends and 32 receives
// are in flight at once with sizes from 8 B to 1 MiB, received sizes are checked, iflush is called
// on the received buffers and every byte is verified against the sender's pattern. Handles travel
// through memory shared by the forked ranks; every wait has a deadline.
// usage: func_ring [plugin.so] [nranks]
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
#include <random>
#include <vector>

#include "nccl_abi.h"

static int g_rank = 0, g_n = 4;
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

using Clock = std::chrono::steady_clock;
static bool expired(Clock::time_point t0, int s = 30) { return Clock::now() - t0 > std::chrono::seconds(s); }

struct Oob {
  char handles[16][NCCL_NET_HANDLE_MAXSIZE];
  std::atomic<int> arrived[64];
  std::atomic<int> failed;
};
static Oob* oob = nullptr;
static int g_barrier_idx = 0;
static int oob_barrier() {
  const int idx = g_barrier_idx++;
  oob->arrived[idx].fetch_add(1);
  const auto t0 = Clock::now();
  while (oob->arrived[idx].load() < g_n) {
    if (oob->failed.load() || expired(t0, 60)) return 1;
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

#include "test_buf.h"

static void fill(std::vector<uint8_t>& b, uint32_t seed) {
  std::mt19937 g(seed);
  for (auto& x : b) x = static_cast<uint8_t>(g());
}

static int run_rank(const char* so) {
  void* h = dlopen(so, RTLD_NOW | RTLD_LOCAL);
  if (!h) FAIL("dlopen: %s", dlerror());
  auto* net = static_cast<ncclNet_v11_t*>(dlsym(h, "ncclNetPlugin_v11"));
  if (!net) FAIL("ncclNetPlugin_v11 not exported");
  void* ctx = nullptr;
  OK(net->init(&ctx, 0x77, nullptr, logger, nullptr));
  void *l = nullptr, *s = nullptr, *r = nullptr;
  OK(net->listen(ctx, 0, oob->handles[g_rank], &l));
  if (oob_barrier()) FAIL("barrier");
  const int next = (g_rank + 1) % g_n, prev = (g_rank + g_n - 1) % g_n;
  auto t0 = Clock::now();
  while (!s || !r) {
    if (!s) OK(net->connect(ctx, 0, oob->handles[next], &s, nullptr));
    if (!r) OK(net->accept(l, &r, nullptr));
    if (expired(t0)) FAIL("ring connect/accept did not finish (s=%p r=%p)", s, r);
  }
  OK(net->closeListen(l));

  const int inflight = 32, rounds = 4;
  const size_t sizes[] = {8, 64, 1000, 4096, 8192, 8200, 65536, 262144 + 3, 1u << 20};
  // host buffers, or device buffers with FUNC_NET_DEVICE=1 and the stand-in driver on the library path
  std::vector<TestBuf> sbuf(inflight), rbuf(inflight);
  std::vector<void*> smh(inflight), rmh(inflight);
  for (int i = 0; i < inflight; ++i) {
    if (buf_alloc(&sbuf[i], 1u << 20) || buf_alloc(&rbuf[i], 1u << 20)) FAIL("buffer allocation failed");
    OK(net->regMr(s, sbuf[i].data(), sbuf[i].size(), buf_type(), &smh[i]));
    OK(net->regMr(r, rbuf[i].data(), rbuf[i].size(), buf_type(), &rmh[i]));
  }
  for (int round = 0; round < rounds; ++round) {
    std::vector<void*> sreq(inflight, nullptr), rreq(inflight, nullptr);
    std::vector<size_t> len(inflight);
    for (int i = 0; i < inflight; ++i) {
      len[i] = sizes[(i + round) % (sizeof(sizes) / sizeof(sizes[0]))];
      std::vector<uint8_t> pattern(len[i]);
      fill(pattern, 1000 * g_rank + 100 * round + i);
      memcpy(sbuf[i].host(), pattern.data(), len[i]);
      memset(rbuf[i].host(), 0xEE, rbuf[i].size());
      if (sbuf[i].to_device(0, len[i]) || rbuf[i].to_device()) FAIL("copy to the device failed");
    }
    // post everything, interleaved, retrying refused posts while the others make progress
    int sp = 0, rp = 0;
    t0 = Clock::now();
    while (sp < inflight || rp < inflight) {
      if (rp < inflight) {
        void* d = rbuf[rp].data();
        size_t cap = rbuf[rp].size();
        int tag = 1;
        OK(net->irecv(r, 1, &d, &cap, &tag, &rmh[rp], nullptr, &rreq[rp]));
        if (rreq[rp]) ++rp;
      }
      if (sp < inflight) {
        OK(net->isend(s, sbuf[sp].data(), len[sp], 1, smh[sp], nullptr, &sreq[sp]));
        if (sreq[sp]) ++sp;
      }
      if (expired(t0)) FAIL("posting stalled in round %d (sent %d, recv %d)", round, sp, rp);
    }
    int left = 2 * inflight;
    std::vector<int> got(inflight, -1);
    t0 = Clock::now();
    while (left) {
      for (int i = 0; i < inflight; ++i) {
        int d = 0, sz = 0;
        if (sreq[i]) {
          OK(net->test(sreq[i], &d, nullptr));
          if (d) {
            sreq[i] = nullptr;
            --left;
          }
        }
        d = 0;
        if (rreq[i]) {
          OK(net->test(rreq[i], &d, &sz));
          if (d) {
            rreq[i] = nullptr;
            got[i] = sz;
            --left;
          }
        }
      }
      if (expired(t0)) FAIL("round %d: %d requests never completed", round, left);
    }
    // flush, then check sizes and bytes against what the previous rank sent
    for (int i = 0; i < inflight; ++i) {
      void* d = rbuf[i].data();
      int sz = got[i];
      void* freq = nullptr;
      OK(net->iflush(r, 1, &d, &sz, &rmh[i], &freq));
      t0 = Clock::now();
      while (freq) {
        int done = 0;
        OK(net->test(freq, &done, nullptr));
        if (done) freq = nullptr;
        if (expired(t0)) FAIL("flush never completed");
      }
      if (got[i] != static_cast<int>(len[i])) FAIL("round %d message %d: received %d bytes, expected %zu", round, i, got[i], len[i]);
      if (rbuf[i].from_device(0, len[i] + 1)) FAIL("copy from the device failed");
      std::vector<uint8_t> want(len[i]);
      fill(want, 1000 * prev + 100 * round + i);
      if (memcmp(want.data(), rbuf[i].host(), len[i])) FAIL("round %d message %d: payload differs", round, i);
      if (len[i] < rbuf[i].size() && rbuf[i].host()[len[i]] != 0xEE) FAIL("round %d message %d: wrote past the message", round, i);
    }
    if (oob_barrier()) FAIL("barrier");
  }
  for (int i = 0; i < inflight; ++i) {
    OK(net->deregMr(s, smh[i]));
    OK(net->deregMr(r, rmh[i]));
    buf_free(&sbuf[i]);
    buf_free(&rbuf[i]);
  }
  OK(net->closeSend(s));
  OK(net->closeRecv(r));
  OK(net->finalize(ctx));
  fprintf(stderr, "[rank %d] ring ok\n", g_rank);
  return 0;
}

int main(int argc, char** argv) {
  const char* so = argc > 1 ? argv[1] : "./libnccl-net-ofi-b200.so";
  g_n = argc > 2 ? atoi(argv[2]) : 4;
  if (g_n < 2 || g_n > 16) return 2;
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
