// Helpers shared by the functional tests that drive the net plugin through its public ABI from two
// forked processes: result macros, a logger, a socket barrier, connect / close of a comm pair and
// deadline-bounded post / wait loops.
#pragma once
#include <dlfcn.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdarg>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "nccl_abi.h"

static int g_rank = 0;
static int g_sock = -1;
static ncclNet_v11_t* net = nullptr;
static void* g_ctx = nullptr;

#define FAIL(...)                                                     \
  do {                                                                \
    fprintf(stderr, "[rank %d] %s:%d: ", g_rank, __FILE__, __LINE__); \
    fprintf(stderr, __VA_ARGS__);                                     \
    fprintf(stderr, "\n");                                            \
    return 1;                                                         \
  } while (0)
#define OK(call)                                                          \
  do {                                                                    \
    ncclResult_t _r = (call);                                             \
    if (_r != ncclSuccess) FAIL("%s returned %d", #call, (int)_r);        \
  } while (0)

using Clock = std::chrono::steady_clock;
static bool expired(Clock::time_point t0, int seconds = 20) { return Clock::now() - t0 > std::chrono::seconds(seconds); }

static void logger(ncclDebugLogLevel level, unsigned long, const char* file, int line, const char* fmt, ...) {
  if (level > NCCL_LOG_WARN && !getenv("FUNC_NET_VERBOSE")) return;
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  fprintf(stderr, "[rank %d] %s (%s:%d)\n", g_rank, buf, file, line);
}

static int xchg(int sock, const void* mine, void* theirs, size_t n) {
  if (write(sock, mine, n) != (ssize_t)n) return 1;
  size_t got = 0;
  while (got < n) {
    ssize_t r = read(sock, (char*)theirs + got, n - got);
    if (r <= 0) return 1;
    got += (size_t)r;
  }
  return 0;
}
static int barrier(int sock) {
  char a = 'b', b = 0;
  return xchg(sock, &a, &b, 1);
}

struct Pair {
  void* l = nullptr;
  void* s = nullptr;
  void* r = nullptr;
};

// Both ranks listen, swap handles and drive connect/accept until both directions are up.
static int connect_pair(int dev, int sock, Pair* p, bool keep_listen = false) {
  char mine[NCCL_NET_HANDLE_MAXSIZE] = {0}, theirs[NCCL_NET_HANDLE_MAXSIZE] = {0};
  OK(net->listen(g_ctx, dev, mine, &p->l));
  if (xchg(sock, mine, theirs, sizeof(mine))) FAIL("handle exchange failed");
  p->s = p->r = nullptr;
  auto t0 = Clock::now();
  while (!p->s || !p->r) {
    if (!p->s) OK(net->connect(g_ctx, dev, theirs, &p->s, nullptr));
    if (!p->r) OK(net->accept(p->l, &p->r, nullptr));
    if (expired(t0)) FAIL("connect/accept did not finish (s=%p r=%p)", p->s, p->r);
  }
  if (!keep_listen) {
    OK(net->closeListen(p->l));
    p->l = nullptr;
  }
  return 0;
}
static int close_pair(Pair* p) {
  if (p->s) OK(net->closeSend(p->s));
  if (p->r) OK(net->closeRecv(p->r));
  if (p->l) OK(net->closeListen(p->l));
  *p = Pair();
  return 0;
}

static int wait_all(std::vector<void*>& reqs, std::vector<int>* sizes_out = nullptr, int nsub = 1) {
  auto t0 = Clock::now();
  std::vector<bool> done(reqs.size(), false);
  size_t ndone = 0;
  if (sizes_out) sizes_out->assign(reqs.size() * nsub, -1);
  while (ndone < reqs.size()) {
    for (size_t i = 0; i < reqs.size(); ++i) {
      if (done[i]) continue;
      int d = 0, sz[8] = {0};
      OK(net->test(reqs[i], &d, sz));
      if (d) {
        done[i] = true;
        ++ndone;
        if (sizes_out)
          for (int k = 0; k < nsub; ++k) (*sizes_out)[i * nsub + k] = sz[k];
      }
    }
    if (expired(t0)) FAIL("requests did not complete: %zu of %zu done", ndone, reqs.size());
  }
  return 0;
}

static void fill(std::vector<uint8_t>& b, uint32_t seed) {
  std::mt19937 g(seed);
  for (auto& x : b) x = (uint8_t)g();
}

// isend / irecv may return a null request: retry with a deadline.
static int post_send(void* s, void* data, size_t n, int tag, void* mh, void** req) {
  auto t0 = Clock::now();
  *req = nullptr;
  while (!*req) {
    OK(net->isend(s, data, n, tag, mh, nullptr, req));
    if (expired(t0)) FAIL("isend kept returning no request (size %zu tag %d)", n, tag);
  }
  return 0;
}
static int post_recv(void* r, int n, void** data, size_t* sizes, int* tags, void** mh, void** req) {
  auto t0 = Clock::now();
  *req = nullptr;
  while (!*req) {
    OK(net->irecv(r, n, data, sizes, tags, mh, nullptr, req));
    if (expired(t0)) FAIL("irecv kept returning no request");
  }
  return 0;
}

