// Functional test of the net plugin through its public ABI only (dlopen + ncclNetPlugin_v11), two
// processes on one host, host or device buffers. Scenarios: connection set-up on every device (1 and 4
// threads), message transfer over a table of (send, recv) sizes incl. truncation with 32 requests
// in flight, the 8 B - 4 MiB ping-pong with tags 0-7 and 8 concurrent requests, grouped receives,
// eager early/late receives, many connections on one listen communicator, close with requests in
// flight, a bandwidth sweep, NCCL's proxy pattern (many channels, one driving thread), transfers
// of device payloads, the table of eager / grouped-receive orderings, dma-buf registrations
// (descriptor and range checks), and the cost of a test() call on a request that is not done. Every poll loop has a
// 20 s deadline; ranks report through exit codes.
// usage: func_net [plugin.so] [scenario]      env: B200NET_* / OFI_NCCL_* parameters apply
//   FUNC_NET_DEVICE=1  payload buffers of the device scenarios (and of proxy_pattern) live in device
//                      memory: on a GPU box through the driver (FUNC_NET_VMM=1 for cuMemCreate
//                      allocations, FUNC_NET_GPU=n to pin the GPU), on a CPU box through the
//                      stand-in driver when it is on the library path (see test_buf.h)
//   FUNC_NET_VERBOSE=1 pass the plugin's INFO lines through
#include <sys/mman.h>

#include <deque>
#include <map>
#include <set>

#include "func_common.h"
#include "test_buf.h"

// ------------------------------------------------------------------------------------------ scenarios
static int scenario_connection(int sock) {
  int ndev = 0;
  OK(net->devices(&ndev));
  if (ndev < 1) FAIL("no devices");
  for (int dev = 0; dev < ndev; ++dev) {
    ncclNetProperties_v11_t props;
    memset(&props, 0, sizeof(props));
    OK(net->getProperties(dev, &props));
    if (!props.name || !(props.ptrSupport & NCCL_PTR_HOST) || props.maxRecvs < 1 || props.maxComms < 1)
      FAIL("implausible properties for device %d", dev);
    Pair p;
    if (connect_pair(dev, sock, &p)) return 1;
    if (close_pair(&p)) return 1;
  }
  return barrier(sock);
}

// regMrDmaBuf: the descriptor has to be open and, where it reports a size, cover offset + size.
// A memfd stands in for a dma-buf descriptor (both answer lseek(SEEK_END) with their size).
static int scenario_dmabuf_registration(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  const int fd = memfd_create("func_net_dmabuf", 0);
  if (fd < 0 || ftruncate(fd, 1 << 16) != 0) FAIL("memfd");
  void* buf = mmap(nullptr, 1 << 16, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (buf == MAP_FAILED) FAIL("mmap");
  void* mh = nullptr;
  OK(net->regMrDmaBuf(p.s, buf, 1 << 16, NCCL_PTR_HOST, 0, fd, &mh));
  if (!mh) FAIL("no handle");
  OK(net->deregMr(p.s, mh));
  OK(net->regMrDmaBuf(p.s, static_cast<char*>(buf) + 4096, 4096, NCCL_PTR_HOST, 4096, fd, &mh));
  OK(net->deregMr(p.s, mh));
  if (net->regMrDmaBuf(p.s, buf, (1 << 16) + 1, NCCL_PTR_HOST, 0, fd, &mh) == ncclSuccess) FAIL("range past the end accepted");
  if (net->regMrDmaBuf(p.s, buf, 4096, NCCL_PTR_HOST, (1 << 16) - 100, fd, &mh) == ncclSuccess) FAIL("offset + size past the end accepted");
  if (net->regMrDmaBuf(p.s, buf, 4096, NCCL_PTR_HOST, 0, -1, &mh) == ncclSuccess) FAIL("descriptor -1 accepted");
  munmap(buf, 1 << 16);
  close(fd);
  if (net->regMrDmaBuf(p.s, buf, 4096, NCCL_PTR_HOST, 0, fd, &mh) == ncclSuccess) FAIL("closed descriptor accepted");
  if (close_pair(&p)) return 1;
  return barrier(sock);
}

static int scenario_message_transfer(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  const size_t pairs[][2] = {{512, 512},       {4096, 4096},         {8192, 8192},       {8200, 16384},
                             {65536, 65536},   {1 << 20, 1 << 20},   {2 << 20, 2 << 20}, {1 << 20, 4096} /* truncated */,
                             {100, 1 << 20},   {0, 64}};
  for (auto& sr : pairs) {
    const size_t ssz = sr[0], rsz = sr[1], expect = ssz < rsz ? ssz : rsz;
    const int NREQ = 32;
    std::vector<std::vector<uint8_t>> sbuf(NREQ, std::vector<uint8_t>(ssz ? ssz : 1)), rbuf(NREQ, std::vector<uint8_t>(rsz, 0xEE));
    void *smh[NREQ], *rmh[NREQ];
    std::vector<void*> reqs;
    for (int i = 0; i < NREQ; ++i) {
      fill(sbuf[i], 1000 * (1 - g_rank) + i);  // what the peer sends to me is seeded with MY rank
      OK(net->regMr(p.s, sbuf[i].data(), sbuf[i].size(), NCCL_PTR_HOST, &smh[i]));
      OK(net->regMr(p.r, rbuf[i].data(), rbuf[i].size(), NCCL_PTR_HOST, &rmh[i]));
    }
    for (int i = 0; i < NREQ; ++i) {
      void* req;
      void* d = rbuf[i].data();
      size_t sz = rsz;
      int tag = 7;
      if (post_recv(p.r, 1, &d, &sz, &tag, &rmh[i], &req)) return 1;
      reqs.push_back(req);
    }
    std::vector<void*> sreqs;
    for (int i = 0; i < NREQ; ++i) {
      void* req;
      if (post_send(p.s, sbuf[i].data(), ssz, 7, smh[i], &req)) return 1;
      sreqs.push_back(req);
    }
    std::vector<int> sizes;
    if (wait_all(reqs, &sizes)) FAIL("receives of pair (%zu,%zu)", ssz, rsz);
    if (wait_all(sreqs)) FAIL("sends of pair (%zu,%zu)", ssz, rsz);
    for (int i = 0; i < NREQ; ++i) {
      if ((size_t)sizes[i] != expect) FAIL("pair (%zu,%zu) req %d: size %d, expected %zu", ssz, rsz, i, sizes[i], expect);
      std::vector<uint8_t> want(ssz ? ssz : 1);
      fill(want, 1000 * g_rank + i);
      if (expect && memcmp(want.data(), rbuf[i].data(), expect)) FAIL("pair (%zu,%zu) req %d: payload differs", ssz, rsz, i);
      if (rsz > expect && rbuf[i][expect] != 0xEE) FAIL("pair (%zu,%zu): bytes past the message were touched", ssz, rsz);
    }
    void* freq;
    void* d0 = rbuf[0].data();
    int fs = (int)expect;
    OK(net->iflush(p.r, 1, &d0, &fs, &rmh[0], &freq));
    if (freq) {
      std::vector<void*> fr{freq};
      if (wait_all(fr)) return 1;
    }
    for (int i = 0; i < NREQ; ++i) {
      OK(net->deregMr(p.s, smh[i]));
      OK(net->deregMr(p.r, rmh[i]));
    }
    if (barrier(sock)) FAIL("barrier");
  }
  return close_pair(&p);
}

// 8 B - 4 MiB, powers of two, uniform random bytes from seed 0, tags 0-7, 8 concurrent requests.
static int scenario_pingpong(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  std::mt19937 gen(0);
  for (size_t sz = 8; sz <= (4u << 20); sz <<= 1) {
    const int NREQ = 8;
    std::vector<std::vector<uint8_t>> payload(NREQ, std::vector<uint8_t>(sz)), rbuf(NREQ, std::vector<uint8_t>(sz));
    for (auto& b : payload)
      for (auto& x : b) x = (uint8_t)gen();  // both ranks draw the same stream: same expected data
    void *smh[NREQ], *rmh[NREQ];
    for (int i = 0; i < NREQ; ++i) {
      OK(net->regMr(p.s, payload[i].data(), sz, NCCL_PTR_HOST, &smh[i]));
      OK(net->regMr(p.r, rbuf[i].data(), sz, NCCL_PTR_HOST, &rmh[i]));
    }
    for (int leg = 0; leg < 2; ++leg) {
      const bool sender = (leg == g_rank);
      std::vector<void*> reqs;
      for (int i = 0; i < NREQ; ++i) {
        void* req;
        if (sender) {
          if (post_send(p.s, payload[i].data(), sz, i, smh[i], &req)) return 1;
        } else {
          void* d = rbuf[i].data();
          size_t s = sz;
          int tag = i;
          memset(d, 0, sz);
          if (post_recv(p.r, 1, &d, &s, &tag, &rmh[i], &req)) return 1;
        }
        reqs.push_back(req);
      }
      std::vector<int> sizes;
      if (wait_all(reqs, &sizes)) return 1;
      if (!sender)
        for (int i = 0; i < NREQ; ++i) {
          if ((size_t)sizes[i] != sz) FAIL("size %zu req %d: got %d bytes", sz, i, sizes[i]);
          if (memcmp(rbuf[i].data(), payload[i].data(), sz)) FAIL("size %zu req %d: payload differs", sz, i);
        }
    }
    for (int i = 0; i < NREQ; ++i) {
      OK(net->deregMr(p.s, smh[i]));
      OK(net->deregMr(p.r, rmh[i]));
    }
  }
  if (barrier(sock)) FAIL("barrier");
  return close_pair(&p);
}

static int scenario_grouped_recv(int sock) {
  ncclNetProperties_v11_t props;
  memset(&props, 0, sizeof(props));
  OK(net->getProperties(0, &props));
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  for (int n : {1, 2, 4, 8}) {
    if (n > props.maxRecvs) continue;
    for (size_t base : {(size_t)64, (size_t)4096, (size_t)(256 << 10)}) {
      // mixed sizes: sub-receive k gets base*(k+1) bytes, tag 100+k; sends go out in reverse tag order
      std::vector<std::vector<uint8_t>> sbuf(n), rbuf(n);
      void* data[8];
      size_t sizes[8];
      int tags[8];
      void *rmh[8], *smh[8];
      for (int k = 0; k < n; ++k) {
        sbuf[k].resize(base * (k + 1));
        rbuf[k].assign(base * (k + 1) + 32, 0);
        fill(sbuf[k], 50 * (1 - g_rank) + k + (uint32_t)base);
        data[k] = rbuf[k].data();
        sizes[k] = rbuf[k].size();
        tags[k] = 100 + k;
        OK(net->regMr(p.r, rbuf[k].data(), rbuf[k].size(), NCCL_PTR_HOST, &rmh[k]));
        OK(net->regMr(p.s, sbuf[k].data(), sbuf[k].size(), NCCL_PTR_HOST, &smh[k]));
      }
      void* rreq;
      if (post_recv(p.r, n, data, sizes, tags, rmh, &rreq)) return 1;
      std::vector<void*> sreqs;
      for (int k = n - 1; k >= 0; --k) {
        void* req;
        if (post_send(p.s, sbuf[k].data(), sbuf[k].size(), 100 + k, smh[k], &req)) return 1;
        sreqs.push_back(req);
      }
      std::vector<void*> rr{rreq};
      std::vector<int> got;
      if (wait_all(rr, &got, n)) return 1;
      if (wait_all(sreqs)) return 1;
      for (int k = 0; k < n; ++k) {
        if ((size_t)got[k] != base * (k + 1)) FAIL("n=%d base=%zu sub %d: size %d", n, base, k, got[k]);
        std::vector<uint8_t> want(base * (k + 1));
        fill(want, 50 * g_rank + k + (uint32_t)base);
        if (memcmp(want.data(), rbuf[k].data(), want.size())) FAIL("n=%d base=%zu sub %d: payload differs", n, base, k);
        OK(net->deregMr(p.r, rmh[k]));
        OK(net->deregMr(p.s, smh[k]));
      }
      if (barrier(sock)) FAIL("barrier");
    }
  }
  return close_pair(&p);
}

// Eager paths: sends posted before any receive exists (early), after it (late), more eager sends
// than the queue holds, the size boundary around the eager limit, and grouped receives fed eagerly.
static int scenario_eager(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  ncclNetProperties_v11_t props;
  memset(&props, 0, sizeof(props));
  OK(net->getProperties(0, &props));
  const char* em = getenv("B200NET_EAGER_MAX_SIZE");
  const bool eager_off = em && atoi(em) == 0;  // with eager disabled nothing can be sent before a receive exists
  for (size_t sz : {(size_t)8, (size_t)1024, (size_t)8191, (size_t)8192, (size_t)8193}) {
    for (int early = 0; early < (eager_off ? 1 : 2); ++early) {
      const int N = 40;  // more than the 32-deep eager queue
      std::vector<std::vector<uint8_t>> sbuf(N, std::vector<uint8_t>(sz)), rbuf(N, std::vector<uint8_t>(sz));
      for (int i = 0; i < N; ++i) fill(sbuf[i], 7 * (1 - g_rank) + i + (uint32_t)sz);
      void* smh;
      void* rmh;
      std::vector<void*> sreqs, rreqs;
      // rank 0 sends first when `early`, rank 1 receives; then roles swap through the barrier order
      auto do_sends = [&](int first, int last) -> int {
        for (int i = first; i < last; ++i) {
          OK(net->regMr(p.s, sbuf[i].data(), sz, NCCL_PTR_HOST, &smh));
          void* req = nullptr;
          auto t0 = Clock::now();
          while (!req) {
            OK(net->isend(p.s, sbuf[i].data(), sz, 3, smh, nullptr, &req));
            // keep earlier sends moving while the queue is full
            for (size_t k = 0; k < sreqs.size(); ++k) {
              if (!sreqs[k]) continue;
              int d = 0;
              OK(net->test(sreqs[k], &d, nullptr));
              if (d) sreqs[k] = nullptr;
            }
            if (expired(t0)) FAIL("eager isend stuck at message %d (size %zu)", i, sz);
          }
          sreqs.push_back(req);
          OK(net->deregMr(p.s, smh));
        }
        return 0;
      };
      auto do_recvs = [&]() -> int {
        for (int i = 0; i < N; ++i) {
          OK(net->regMr(p.r, rbuf[i].data(), sz, NCCL_PTR_HOST, &rmh));
          void* d = rbuf[i].data();
          size_t s = sz;
          int tag = 3;
          void* req;
          if (post_recv(p.r, 1, &d, &s, &tag, &rmh, &req)) return 1;
          rreqs.push_back(req);
          OK(net->deregMr(p.r, rmh));
        }
        return 0;
      };
      if (early) {
        // only 32 eager sends may be outstanding with no receive posted: the 33rd must be refused
        // (null request) until the receiver shows up
        // (the tagged protocol has no such window: it buffers at the receiver, so it sends all at once)
        const bool windowed = props.maxRecvs > 1;
        const int first_batch = !windowed ? N : (sz <= 8192 ? 32 : 0);
        if (g_rank == 0 && do_sends(0, first_batch)) return 1;
        if (g_rank == 0 && first_batch && windowed) {
          void* extra = nullptr;
          OK(net->regMr(p.s, sbuf[first_batch].data(), sz, NCCL_PTR_HOST, &smh));
          OK(net->isend(p.s, sbuf[first_batch].data(), sz, 3, smh, nullptr, &extra));
          OK(net->deregMr(p.s, smh));
          if (extra) FAIL("a 33rd eager send was accepted with no receive posted");
        }
        if (barrier(sock)) FAIL("barrier");
        if (g_rank == 1 && do_recvs()) return 1;
        if (g_rank == 0 && do_sends(first_batch, N)) return 1;
      } else {
        if (g_rank == 1 && do_recvs()) return 1;
        if (barrier(sock)) FAIL("barrier");
        if (g_rank == 0 && do_sends(0, N)) return 1;
      }
      std::vector<void*> live;
      for (void* r : sreqs)
        if (r) live.push_back(r);
      // both ranks must keep polling: the sender's eager requests finish when control messages arrive
      std::vector<int> sizes;
      if (g_rank == 1) {
        if (wait_all(rreqs, &sizes)) return 1;
        for (int i = 0; i < N; ++i) {
          std::vector<uint8_t> want(sz);
          fill(want, 7 * g_rank + i + (uint32_t)sz);
          if ((size_t)sizes[i] != sz || memcmp(want.data(), rbuf[i].data(), sz))
            FAIL("eager size %zu early=%d msg %d: wrong size (%d) or payload", sz, early, i, sizes[i]);
        }
      } else {
        if (wait_all(live)) return 1;
      }
      if (barrier(sock)) FAIL("barrier");
    }
  }
  // grouped receive fed by eager sends that were posted first (all-eager group, mixed tags)
  if (props.maxRecvs >= 4 && !eager_off) {
    const int n = 4;
    std::vector<std::vector<uint8_t>> sbuf(n, std::vector<uint8_t>(512)), rbuf(n, std::vector<uint8_t>(512));
    std::vector<void*> sreqs;
    void* mh[4];
    if (g_rank == 0) {
      for (int k = 0; k < n; ++k) {
        fill(sbuf[k], 900 + k);
        void* req;
        OK(net->regMr(p.s, sbuf[k].data(), 512, NCCL_PTR_HOST, &mh[k]));
        if (post_send(p.s, sbuf[k].data(), 512, 20 + (k % 2), mh[k], &req)) return 1;
        sreqs.push_back(req);
      }
    }
    if (barrier(sock)) FAIL("barrier");
    if (g_rank == 1) {
      void* data[4];
      size_t sizes[4];
      int tags[4] = {20, 21, 20, 21};
      void* rmh[4];
      for (int k = 0; k < n; ++k) {
        data[k] = rbuf[k].data();
        sizes[k] = 512;
        OK(net->regMr(p.r, rbuf[k].data(), 512, NCCL_PTR_HOST, &rmh[k]));
      }
      void* req;
      if (post_recv(p.r, n, data, sizes, tags, rmh, &req)) return 1;
      std::vector<void*> rr{req};
      std::vector<int> got;
      if (wait_all(rr, &got, n)) return 1;
      // sends in order: tags 20,21,20,21 -> entries 0,1,2,3
      for (int k = 0; k < n; ++k) {
        std::vector<uint8_t> want(512);
        fill(want, 900 + k);
        if (got[k] != 512 || memcmp(want.data(), rbuf[k].data(), 512)) FAIL("eager group: sub %d wrong", k);
        OK(net->deregMr(p.r, rmh[k]));
      }
    } else {
      if (wait_all(sreqs)) return 1;
      for (int k = 0; k < n; ++k) OK(net->deregMr(p.s, mh[k]));
    }
    if (barrier(sock)) FAIL("barrier");
  }
  return close_pair(&p);
}

static int scenario_reuse_listen(int sock) {
  Pair base;
  char mine[NCCL_NET_HANDLE_MAXSIZE] = {0}, theirs[NCCL_NET_HANDLE_MAXSIZE] = {0};
  OK(net->listen(g_ctx, 0, mine, &base.l));
  if (xchg(sock, mine, theirs, sizeof(mine))) FAIL("handle exchange");
  for (int round = 0; round < 12; ++round) {
    char h[NCCL_NET_HANDLE_MAXSIZE];
    memcpy(h, theirs, sizeof(h));  // a fresh copy: connect keeps its progress inside the handle
    void *s = nullptr, *r = nullptr;
    auto t0 = Clock::now();
    while (!s || !r) {
      if (!s) OK(net->connect(g_ctx, 0, h, &s, nullptr));
      if (!r) OK(net->accept(base.l, &r, nullptr));
      if (expired(t0)) FAIL("round %d: connect/accept stuck", round);
    }
    uint64_t out = 0xabc000 + round + g_rank, in = 0;
    void *smh, *rmh, *sreq, *rreq;
    OK(net->regMr(s, &out, sizeof(out), NCCL_PTR_HOST, &smh));
    OK(net->regMr(r, &in, sizeof(in), NCCL_PTR_HOST, &rmh));
    void* d = &in;
    size_t sz = sizeof(in);
    int tag = 1;
    if (post_recv(r, 1, &d, &sz, &tag, &rmh, &rreq)) return 1;
    if (post_send(s, &out, sizeof(out), 1, smh, &sreq)) return 1;
    std::vector<void*> reqs{rreq, sreq};
    if (wait_all(reqs)) return 1;
    if (in != 0xabc000u + round + (1 - g_rank)) FAIL("round %d: got %llx", round, (unsigned long long)in);
    OK(net->deregMr(s, smh));
    OK(net->deregMr(r, rmh));
    if (barrier(sock)) FAIL("barrier");
    OK(net->closeSend(s));
    OK(net->closeRecv(r));
  }
  OK(net->closeListen(base.l));
  return barrier(sock);
}

// Close communicators while 32 receives are still posted and unmatched: no crash, no hang, and a
// fresh connection works afterwards (the aborted endpoint is replaced).
static int scenario_inflight_close(int sock) {
  for (int iter = 0; iter < 10; ++iter) {
    Pair p;
    if (connect_pair(0, sock, &p)) return 1;
    const int N = 32;
    std::vector<std::vector<uint8_t>> rbuf(N, std::vector<uint8_t>(1 << 16));
    std::vector<void*> mhs(N);
    for (int i = 0; i < N; ++i) {
      OK(net->regMr(p.r, rbuf[i].data(), rbuf[i].size(), NCCL_PTR_HOST, &mhs[i]));
      void* d = rbuf[i].data();
      size_t s = rbuf[i].size();
      int tag = 0;
      void* req;
      if (post_recv(p.r, 1, &d, &s, &tag, &mhs[i], &req)) return 1;
    }
    if (barrier(sock)) FAIL("barrier");
    for (int i = 0; i < N; ++i) OK(net->deregMr(p.r, mhs[i]));
    OK(net->closeRecv(p.r));
    OK(net->closeSend(p.s));
    p = Pair();
    if (barrier(sock)) FAIL("barrier");
  }
  Pair q;
  if (connect_pair(0, sock, &q)) return 1;
  return close_pair(&q);
}


// Sizes around the eager limit and up to several stripes, every message checked byte for byte,
// several in flight; in device mode this walks the eager-pack path (small), the copy kernel
// (large) and the receiver's copy of early eager payloads into device memory.
static int scenario_device_transfer(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  const size_t sizes[] = {0, 1, 8, 100, 4096, 8192, 8193, 65536, 300000, 1u << 20, (4u << 20) + 16};
  const int nmsg = sizeof(sizes) / sizeof(sizes[0]);
  size_t eager_limit = 8192;   // the plugin's default; the suite also runs with eager switched off
  for (const char* name : {"B200NET_EAGER_MAX_SIZE", "OFI_NCCL_EAGER_MAX_SIZE"})
    if (const char* v = getenv(name)) eager_limit = strtoull(v, nullptr, 0);
  for (int pass = 0; pass < 2; ++pass) {   // pass 0: receives first; pass 1: sends first (early eager)
    std::vector<TestBuf> sb(nmsg), rb(nmsg);
    std::vector<void*> smh(nmsg), rmh(nmsg), sreq(nmsg, nullptr), rreq(nmsg, nullptr);
    for (int i = 0; i < nmsg; ++i) {
      if (buf_alloc(&sb[i], sizes[i] + 64) || buf_alloc(&rb[i], sizes[i] + 64)) FAIL("buffer allocation failed");
      std::vector<uint8_t> pat(sizes[i]);
      fill(pat, 500 + 10 * pass + i + 1000 * g_rank);
      if (sizes[i]) memcpy(sb[i].host(), pat.data(), sizes[i]);
      memset(rb[i].host(), 0xCD, rb[i].size());
      if (sb[i].to_device() || rb[i].to_device()) FAIL("copy to the device failed");
      OK(net->regMr(p.s, sb[i].data(), sb[i].size(), buf_type(), &smh[i]));
      OK(net->regMr(p.r, rb[i].data(), rb[i].size(), buf_type(), &rmh[i]));
    }
    if (barrier(sock)) FAIL("barrier");
    auto post_recvs = [&]() -> int {
      for (int i = 0; i < nmsg; ++i) {
        void* d = rb[i].data();
        size_t cap = sizes[i];
        int tag = 7;
        if (post_recv(p.r, 1, &d, &cap, &tag, &rmh[i], &rreq[i])) return 1;
      }
      return 0;
    };
    auto post_sends = [&]() -> int {
      for (int i = 0; i < nmsg; ++i) {
        auto t0 = Clock::now();
        while (!sreq[i]) {
          OK(net->isend(p.s, sb[i].data(), sizes[i], 7, smh[i], nullptr, &sreq[i]));
          if (!sreq[i] && pass == 1 && (sizes[i] > eager_limit || sizes[i] > 8192 || eager_limit == 0)) break;   // no receive yet and not eager: later
          if (expired(t0)) FAIL("isend of %zu bytes kept returning no request", sizes[i]);
        }
      }
      return 0;
    };
    if (pass == 0) {
      if (post_recvs()) return 1;
      if (barrier(sock)) FAIL("barrier");
      if (post_sends()) return 1;
    } else {
      if (post_sends()) return 1;   // eager-sized ones go out with no receive posted
      if (barrier(sock)) FAIL("barrier");
      if (post_recvs()) return 1;
      for (int i = 0; i < nmsg; ++i) {
        auto t0 = Clock::now();
        while (!sreq[i]) {
          OK(net->isend(p.s, sb[i].data(), sizes[i], 7, smh[i], nullptr, &sreq[i]));
          if (expired(t0)) FAIL("late isend of %zu bytes kept returning no request", sizes[i]);
        }
      }
    }
    std::vector<void*> all;
    for (void* r : sreq) all.push_back(r);
    for (void* r : rreq) all.push_back(r);
    std::vector<int> got;
    if (wait_all(all, &got)) return 1;
    {   // what NCCL does before its kernel reads received device data: a flush over the receive buffers
      std::vector<void*> fd(nmsg);
      std::vector<int> fs(nmsg);
      for (int i = 0; i < nmsg; ++i) {
        fd[i] = rb[i].data();
        fs[i] = static_cast<int>(sizes[i]);
      }
      void* freq = nullptr;
      OK(net->iflush(p.r, std::min(nmsg, 8), fd.data(), fs.data(), rmh.data(), &freq));
      if (freq) {
        std::vector<void*> fr{freq};
        if (wait_all(fr)) return 1;
      }
    }
    for (int i = 0; i < nmsg; ++i) {
      std::vector<uint8_t> want(sizes[i]);
      fill(want, 500 + 10 * pass + i + 1000 * (1 - g_rank));
      if (got[nmsg + i] != static_cast<int>(sizes[i])) FAIL("pass %d message %d: size %d, expected %zu", pass, i, got[nmsg + i], sizes[i]);
      if (rb[i].from_device()) FAIL("copy from the device failed");
      if (sizes[i] && memcmp(want.data(), rb[i].host(), sizes[i])) {
        size_t at = 0;
        while (at < sizes[i] && want[at] == rb[i].host()[at]) ++at;
        FAIL("pass %d message %d (%zu bytes): payload differs from byte %zu on: got %02x %02x %02x %02x, expected %02x %02x %02x %02x "
             "(cd = never written, 00 = zero-filled)", pass, i, sizes[i], at, rb[i].host()[at], rb[i].host()[std::min(at + 1, sizes[i] - 1)],
             rb[i].host()[std::min(at + 2, sizes[i] - 1)], rb[i].host()[std::min(at + 3, sizes[i] - 1)], want[at],
             want[std::min(at + 1, sizes[i] - 1)], want[std::min(at + 2, sizes[i] - 1)], want[std::min(at + 3, sizes[i] - 1)]);
      }
      if (rb[i].host()[sizes[i]] != 0xCD) FAIL("pass %d message %d: wrote past the end", pass, i);
    }
    if (barrier(sock)) FAIL("barrier");
    for (int i = 0; i < nmsg; ++i) {
      OK(net->deregMr(p.s, smh[i]));
      OK(net->deregMr(p.r, rmh[i]));
      buf_free(&sb[i]);
      buf_free(&rb[i]);
    }
  }
  return close_pair(&p);
}

// The access pattern of NCCL's proxy thread: several channels, each a connection in both
// directions, every channel keeps up to eight receives posted and eight chunk-sized sends in
// flight, and ONE thread per process drives all of them round-robin with isend / irecv / test,
// never blocking on any single request. Every chunk carries its channel and step in its first
// bytes and is checked on arrival.
static int scenario_proxy_pattern(int sock) {
  const int channels = getenv("FUNC_NET_PROXY_CHANNELS") ? atoi(getenv("FUNC_NET_PROXY_CHANNELS")) : 8;
  const int steps = 8;
  const int chunks_per_channel = getenv("FUNC_NET_PROXY_CHUNKS") ? atoi(getenv("FUNC_NET_PROXY_CHUNKS")) : 48;
  const size_t chunk = getenv("FUNC_NET_PROXY_CHUNK") ? strtoul(getenv("FUNC_NET_PROXY_CHUNK"), nullptr, 0) : (1u << 20);
  struct Chan {
    Pair p;
    std::vector<TestBuf> sbuf, rbuf;
    std::vector<void*> smh, rmh, sreq, rreq;
    std::vector<int> rreq_chunk, sreq_chunk;
    int sent = 0, send_done = 0, posted = 0, recv_done = 0;
  };
  std::vector<Chan> ch(channels);
  for (int c = 0; c < channels; ++c) {
    if (connect_pair(0, sock, &ch[c].p)) return 1;
    ch[c].sbuf.assign(steps, TestBuf());
    ch[c].rbuf.assign(steps, TestBuf());
    for (int s = 0; s < steps; ++s)
      if (buf_alloc(&ch[c].sbuf[s], chunk) || buf_alloc(&ch[c].rbuf[s], chunk)) FAIL("buffer allocation failed");
    ch[c].smh.assign(steps, nullptr);
    ch[c].rmh.assign(steps, nullptr);
    ch[c].sreq.assign(steps, nullptr);
    ch[c].rreq.assign(steps, nullptr);
    ch[c].rreq_chunk.assign(steps, -1);
    ch[c].sreq_chunk.assign(steps, -1);
    for (int s = 0; s < steps; ++s) {
      OK(net->regMr(ch[c].p.s, ch[c].sbuf[s].data(), chunk, buf_type(), &ch[c].smh[s]));
      OK(net->regMr(ch[c].p.r, ch[c].rbuf[s].data(), chunk, buf_type(), &ch[c].rmh[s]));
    }
  }
  if (barrier(sock)) FAIL("barrier");
  auto stamp = [&](TestBuf& b, int c, int k) {
    uint32_t hdr[4] = {0xC0FFEEu, static_cast<uint32_t>(g_rank), static_cast<uint32_t>(c), static_cast<uint32_t>(k)};
    memcpy(b.host(), hdr, sizeof(hdr));
    b.host()[chunk - 1] = static_cast<uint8_t>(c * 31 + k);
    b.to_device(0, sizeof(hdr));
    b.to_device(chunk - 1, 1);
  };
  auto t0 = Clock::now();
  long done_total = 0, calls = 0;
  const long want_total = 2L * channels * chunks_per_channel;
  while (done_total < want_total) {
    for (int c = 0; c < channels; ++c) {
      Chan& x = ch[c];
      // keep receives posted ahead
      while (x.posted < chunks_per_channel && x.posted - x.recv_done < steps) {
        const int slot = x.posted % steps;
        void* d = x.rbuf[slot].data();
        size_t sz = chunk;
        int tag = c;
        void* req = nullptr;
        OK(net->irecv(x.p.r, 1, &d, &sz, &tag, &x.rmh[slot], nullptr, &req));
        ++calls;
        if (!req) break;
        x.rreq[slot] = req;
        x.rreq_chunk[slot] = x.posted++;
      }
      // keep sends in flight
      while (x.sent < chunks_per_channel && x.sent - x.send_done < steps) {
        const int slot = x.sent % steps;
        stamp(x.sbuf[slot], c, x.sent);
        void* req = nullptr;
        OK(net->isend(x.p.s, x.sbuf[slot].data(), chunk, c, x.smh[slot], nullptr, &req));
        ++calls;
        if (!req) break;
        x.sreq[slot] = req;
        x.sreq_chunk[slot] = x.sent++;
      }
      // poll the oldest outstanding request of each kind (NCCL completes them in order)
      if (x.send_done < x.sent) {
        const int slot = x.send_done % steps;
        int d = 0;
        OK(net->test(x.sreq[slot], &d, nullptr));
        ++calls;
        if (d) {
          ++x.send_done;
          ++done_total;
        }
      }
      if (x.recv_done < x.posted) {
        const int slot = x.recv_done % steps;
        int d = 0, sz = 0;
        OK(net->test(x.rreq[slot], &d, &sz));
        ++calls;
        if (d) {
          uint32_t hdr[4];
          x.rbuf[slot].from_device(0, sizeof(hdr));
          x.rbuf[slot].from_device(chunk - 1, 1);
          memcpy(hdr, x.rbuf[slot].host(), sizeof(hdr));
          const int k = x.rreq_chunk[slot];
          if (sz != static_cast<int>(chunk) || hdr[0] != 0xC0FFEEu || hdr[1] != static_cast<uint32_t>(1 - g_rank) ||
              hdr[2] != static_cast<uint32_t>(c) || hdr[3] != static_cast<uint32_t>(k) ||
              x.rbuf[slot].host()[chunk - 1] != static_cast<uint8_t>(c * 31 + k))
            FAIL("channel %d chunk %d arrived wrong (size %d, hdr %x %u %u %u)", c, k, sz, hdr[0], hdr[1], hdr[2], hdr[3]);
          ++x.recv_done;
          ++done_total;
        }
      }
    }
    if (expired(t0, 60)) {
      for (int c = 0; c < channels; ++c)
        fprintf(stderr, "[rank %d] channel %d: sent %d/%d done, posted %d recv done %d\n", g_rank, c, ch[c].sent, ch[c].send_done,
                ch[c].posted, ch[c].recv_done);
      FAIL("proxy pattern stalled at %ld of %ld completions", done_total, want_total);
    }
  }
  if (g_rank == 0) {
    const double secs = std::chrono::duration<double>(Clock::now() - t0).count();
    fprintf(stderr, "[rank 0] proxy pattern: %.2f GB/s per direction (%d channels x %d chunks of %zu KiB in %.3f s; %ld plugin "
            "calls, %.0f ns of the loop per call)\n",
            static_cast<double>(channels) * chunks_per_channel * chunk / secs / 1e9, channels, chunks_per_channel, chunk >> 10, secs,
            calls, secs * 1e9 / static_cast<double>(calls));
  }
  if (barrier(sock)) FAIL("barrier");
  for (int c = 0; c < channels; ++c) {
    for (int s = 0; s < steps; ++s) {
      OK(net->deregMr(ch[c].p.s, ch[c].smh[s]));
      OK(net->deregMr(ch[c].p.r, ch[c].rmh[s]));
      buf_free(&ch[c].sbuf[s]);
      buf_free(&ch[c].rbuf[s]);
    }
    if (close_pair(&ch[c].p)) return 1;
  }
  return 0;
}

// What one call of test() costs on a request that is not done yet (NCCL's proxy thread makes
// thousands of them per collective): a receive is posted and tested 2 million times before its
// send is posted; then a send whose receive is not posted yet. Prints nanoseconds per call.
static int scenario_test_call_cost(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  const size_t n = 65536;
  TestBuf sb, rb;
  if (buf_alloc(&sb, n) || buf_alloc(&rb, n)) FAIL("buffer allocation failed");
  void *smh = nullptr, *rmh = nullptr;
  OK(net->regMr(p.s, sb.data(), n, buf_type(), &smh));
  OK(net->regMr(p.r, rb.data(), n, buf_type(), &rmh));
  const int calls = getenv("FUNC_NET_TEST_CALLS") ? atoi(getenv("FUNC_NET_TEST_CALLS")) : 2000000;
  void* data = rb.data();
  size_t sz = n;
  int tag = 3;
  void* rreq = nullptr;
  if (post_recv(p.r, 1, &data, &sz, &tag, &rmh, &rreq)) return 1;
  auto t0 = Clock::now();
  int done = 0, szs[8];
  for (int i = 0; i < calls && !done; ++i) OK(net->test(rreq, &done, szs));
  const double recv_ns = std::chrono::duration<double>(Clock::now() - t0).count() * 1e9 / calls;
  if (done) FAIL("the receive completed although nothing was sent");
  if (barrier(sock)) FAIL("barrier");   // both ranks have measured: now the sends may go
  void* sreq = nullptr;
  if (post_send(p.s, sb.data(), n, 3, smh, &sreq)) return 1;
  std::vector<void*> reqs{sreq, rreq};
  if (wait_all(reqs)) return 1;
  if (g_rank == 0) fprintf(stderr, "[rank 0] test() on a pending receive: %.0f ns per call\n", recv_ns);
  OK(net->deregMr(p.s, smh));
  OK(net->deregMr(p.r, rmh));
  buf_free(&sb);
  buf_free(&rb);
  if (close_pair(&p)) return 1;
  return barrier(sock);
}

// Large rendezvous messages, eight in flight: reports the one-way bandwidth of the host path.
static int scenario_bandwidth(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  const size_t n = 16u << 20;
  const int rounds = 6, window = 8;
  std::vector<std::vector<uint8_t>> bufs(window, std::vector<uint8_t>(n));
  for (int i = 0; i < window; ++i) fill(bufs[i], 100 + i + 50 * g_rank);
  std::vector<void*> mhs(window);
  void* comm = g_rank == 0 ? p.s : p.r;
  for (int i = 0; i < window; ++i) OK(net->regMr(comm, bufs[i].data(), n, NCCL_PTR_HOST, &mhs[i]));
  if (barrier(sock)) FAIL("barrier");
  const auto t0 = Clock::now();
  for (int r = 0; r < rounds; ++r) {
    std::vector<void*> reqs(window);
    for (int i = 0; i < window; ++i) {
      if (g_rank == 0) {
        if (post_send(p.s, bufs[i].data(), n, 9, mhs[i], &reqs[i])) return 1;
      } else {
        void* d = bufs[i].data();
        size_t sz = n;
        int tag = 9;
        if (post_recv(p.r, 1, &d, &sz, &tag, &mhs[i], &reqs[i])) return 1;
      }
    }
    if (wait_all(reqs)) return 1;
  }
  const double secs = std::chrono::duration<double>(Clock::now() - t0).count();
  if (g_rank == 1) {
    for (int i = 0; i < window; ++i) {
      std::vector<uint8_t> want(n);
      fill(want, 100 + i);
      if (bufs[i] != want) FAIL("payload %d differs after the bandwidth run", i);
    }
    fprintf(stderr, "[rank 1] bandwidth: %.2f GB/s one way (%d x %d x %zu MiB in %.3f s)\n",
            rounds * window * static_cast<double>(n) / secs / 1e9, rounds, window, n >> 20, secs);
  }
  for (int i = 0; i < window; ++i) OK(net->deregMr(comm, mhs[i]));
  return close_pair(&p);
}

// One-way throughput of isend / irecv / test on buffers of the mode under test (device memory with
// FUNC_NET_DEVICE=1: the copy kernel over NVLink when the two ranks sit on two GPUs), for several
// message sizes with eight messages in flight. Prints one line per size on rank 1; the last
// window of every size is checked byte for byte.
static int scenario_device_bandwidth(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  const int window = 8;
  const size_t max_n = getenv("FUNC_NET_BW_MAX") ? strtoull(getenv("FUNC_NET_BW_MAX"), nullptr, 0) : (32u << 20);
  std::vector<TestBuf> bufs(window);
  std::vector<void*> mhs(window);
  void* comm = g_rank == 0 ? p.s : p.r;
  for (int i = 0; i < window; ++i) {
    if (buf_alloc(&bufs[i], max_n)) FAIL("buffer allocation failed");
    std::vector<uint8_t> pat(max_n);
    fill(pat, 300 + i + 50 * g_rank);
    memcpy(bufs[i].host(), pat.data(), max_n);
    if (bufs[i].to_device()) FAIL("copy to the device failed");
    OK(net->regMr(comm, bufs[i].data(), max_n, buf_type(), &mhs[i]));
  }
  for (size_t n = 64u << 10; n <= max_n; n *= 4) {
    const int rounds = n >= (8u << 20) ? 12 : 40;
    if (barrier(sock)) FAIL("barrier");
    double secs = 0;
    for (int r = -2; r < rounds; ++r) {   // two warm-up rounds (first use maps the peer's buffers)
      const auto t0 = Clock::now();
      std::vector<void*> reqs(window);
      for (int i = 0; i < window; ++i) {
        if (g_rank == 0) {
          if (post_send(p.s, bufs[i].data(), n, 9, mhs[i], &reqs[i])) return 1;
        } else {
          void* d = bufs[i].data();
          size_t sz = n;
          int tag = 9;
          if (post_recv(p.r, 1, &d, &sz, &tag, &mhs[i], &reqs[i])) return 1;
        }
      }
      if (wait_all(reqs)) return 1;
      if (r >= 0) secs += std::chrono::duration<double>(Clock::now() - t0).count();
    }
    if (g_rank == 1) {
      for (int i = 0; i < window; ++i) {
        std::vector<uint8_t> want(max_n);
        fill(want, 300 + i);
        if (bufs[i].from_device(0, n)) FAIL("copy from the device failed");
        if (memcmp(bufs[i].host(), want.data(), n)) FAIL("payload %d of %zu bytes differs after the bandwidth run", i, n);
      }
      fprintf(stderr, "[rank 1] %s bandwidth %8zu KiB x %d in flight: %8.2f GB/s one way, %7.1f us per message\n",
              device_mode() ? "device" : "host", n >> 10, window, rounds * window * static_cast<double>(n) / secs / 1e9,
              secs / (rounds * window) * 1e6);
    }
  }
  for (int i = 0; i < window; ++i) {
    OK(net->deregMr(comm, mhs[i]));
    buf_free(&bufs[i]);
  }
  return close_pair(&p);
}

// Several thousand messages over ONE connection, so that the 10-bit message sequence numbers, the
// 16-bit eager sequence numbers' low bits and the mailbox slots all wrap several times, with eight
// messages in flight, sizes that alternate between eager and rendezvous, and every payload checked.
static int scenario_seq_wrap(int sock) {
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  const int total = getenv("FUNC_NET_WRAP_MESSAGES") ? atoi(getenv("FUNC_NET_WRAP_MESSAGES")) : 5000, window = 8;
  const size_t sizes[] = {64, 40000, 24, 300000, 4096, 9000};
  const size_t cap = 300000;
  size_t eager_limit = 8192;   // the plugin's default; the suite also runs with eager switched off
  for (const char* name : {"B200NET_EAGER_MAX_SIZE", "OFI_NCCL_EAGER_MAX_SIZE"})
    if (const char* v = getenv(name)) eager_limit = strtoull(v, nullptr, 0);
  eager_limit = std::min<size_t>(eager_limit, 8192);
  std::vector<TestBuf> sb(window), rb(window);
  std::vector<void*> smh(window), rmh(window);
  for (int i = 0; i < window; ++i) {
    if (buf_alloc(&sb[i], cap) || buf_alloc(&rb[i], cap)) FAIL("buffer allocation failed");
    OK(net->regMr(p.s, sb[i].data(), cap, buf_type(), &smh[i]));
    OK(net->regMr(p.r, rb[i].data(), cap, buf_type(), &rmh[i]));
  }
  if (barrier(sock)) FAIL("barrier");
  for (int base = 0; base < total; base += window) {
    std::vector<void*> reqs;
    std::vector<bool> sent(window, false);
    // odd rounds post the sends first, so that eager-sized ones leave before their receive exists
    const int mode = getenv("FUNC_NET_WRAP_MODE") ? atoi(getenv("FUNC_NET_WRAP_MODE")) : 0;   // 1: receives always first, 2: sends always first
    const bool sends_first = mode == 1 ? false : mode == 2 ? true : ((base / window) & 1);
    for (int phase = 0; phase < 2; ++phase) {
      const bool do_sends = (phase == 0) == sends_first;
      for (int i = 0; i < window && base + i < total; ++i) {
        const int k = base + i;
        const size_t n = sizes[k % 6];
        void* req = nullptr;
        if (do_sends) {
          uint32_t hdr[2] = {0xABCD0000u + static_cast<uint32_t>(g_rank), static_cast<uint32_t>(k)};
          memcpy(sb[i].host(), hdr, 8);
          sb[i].host()[n - 1] = static_cast<uint8_t>(k * 7 + g_rank);
          sb[i].to_device(0, 8);
          sb[i].to_device(n - 1, 1);
          auto t0 = Clock::now();
          while (!req) {
            OK(net->isend(p.s, sb[i].data(), n, i, smh[i], nullptr, &req));
            if (!req && sends_first && n > eager_limit) break;   // not eager and no receive yet: after the receives
            if (expired(t0)) FAIL("isend %d kept returning no request", k);
          }
          if (req) {
            reqs.push_back(req);
            sent[i] = true;
          }
        } else {
          void* d = rb[i].data();
          size_t sz = n;
          int tag = i;   // one tag per slot: a round's messages may be sent in another order than its receives are posted
          if (post_recv(p.r, 1, &d, &sz, &tag, &rmh[i], &req)) return 1;
          reqs.push_back(req);
        }
      }
    }
    if (sends_first) {   // the sends that had to wait for their receive
      for (int i = 0; i < window && base + i < total; ++i) {
        const size_t n = sizes[(base + i) % 6];
        if (sent[i]) continue;   // went out before the receives (eager, or its receive was already there)
        void* req = nullptr;
        if (post_send(p.s, sb[i].data(), n, i, smh[i], &req)) return 1;
        reqs.push_back(req);
      }
    }
    if (wait_all(reqs)) return 1;
    for (int i = 0; i < window && base + i < total; ++i) {
      const int k = base + i;
      const size_t n = sizes[k % 6];
      rb[i].from_device(0, 8);
      rb[i].from_device(n - 1, 1);
      uint32_t hdr[2];
      memcpy(hdr, rb[i].host(), 8);
      if (hdr[0] != 0xABCD0000u + static_cast<uint32_t>(1 - g_rank) || hdr[1] != static_cast<uint32_t>(k) ||
          rb[i].host()[n - 1] != static_cast<uint8_t>(k * 7 + (1 - g_rank)))
        FAIL("message %d (%zu bytes) arrived as %x / %u", k, n, hdr[0], hdr[1]);
    }
  }
  for (int i = 0; i < window; ++i) {
    OK(net->deregMr(p.s, smh[i]));
    OK(net->deregMr(p.r, rmh[i]));
    buf_free(&sb[i]);
    buf_free(&rb[i]);
  }
  return close_pair(&p);
}

static int scenario_threads(int) {
  // each thread gets its own endpoint: 4 threads connect to themselves (loopback) concurrently
  std::vector<std::thread> th;
  std::vector<int> rc(4, 1);
  for (int t = 0; t < 4; ++t) {
    th.emplace_back([&, t]() {
      char h[NCCL_NET_HANDLE_MAXSIZE] = {0};
      void *l = nullptr, *s = nullptr, *r = nullptr;
      if (net->listen(g_ctx, 0, h, &l) != ncclSuccess) return;
      auto t0 = Clock::now();
      while ((!s || !r) && !expired(t0)) {
        if (!s && net->connect(g_ctx, 0, h, &s, nullptr) != ncclSuccess) return;
        if (!r && net->accept(l, &r, nullptr) != ncclSuccess) return;
      }
      if (!s || !r) return;
      uint64_t out = 77 + t, in = 0;
      void *smh, *rmh, *sreq = nullptr, *rreq = nullptr;
      net->regMr(s, &out, 8, NCCL_PTR_HOST, &smh);
      net->regMr(r, &in, 8, NCCL_PTR_HOST, &rmh);
      void* d = &in;
      size_t sz = 8;
      int tag = 5;
      while (!rreq && !expired(t0)) net->irecv(r, 1, &d, &sz, &tag, &rmh, nullptr, &rreq);
      while (!sreq && !expired(t0)) net->isend(s, &out, 8, 5, smh, nullptr, &sreq);
      int ds = 0, dr = 0;
      while ((!ds || !dr) && !expired(t0)) {
        if (!ds) net->test(sreq, &ds, nullptr);
        if (!dr) net->test(rreq, &dr, nullptr);
      }
      net->deregMr(s, smh);
      net->deregMr(r, rmh);
      net->closeSend(s);
      net->closeRecv(r);
      net->closeListen(l);
      if (ds && dr && in == 77u + t) rc[t] = 0;
    });
  }
  for (auto& t : th) t.join();
  for (int t = 0; t < 4; ++t)
    if (rc[t]) FAIL("thread %d failed", t);
  return 0;
}

// Eager and rendezvous sends against single and grouped receives in every order that the tag
// rules allow (the cases of the reference's tests/functional/eager_multirecv.cpp:105-1652, as a
// table): per tag, the k-th send must land in the k-th posted entry of that tag, whatever the
// interleaving, whether it travelled eagerly or as a write, and whether the receives were posted
// before or after the sends. The sender posts the way NCCL does: a refused send (null request)
// holds back later sends of the same tag in that round, other tags go on.
struct EmrSend {
  int tag;
  bool large;
};
struct EmrCase {
  const char* name;
  std::vector<EmrSend> sends;
  std::vector<std::vector<int>> groups;   // tags of each posted receive, in posting order
};

static int run_emr_case(const EmrCase& c, Pair& p, int sock, bool late, int max_recvs) {
  for (const auto& g : c.groups)
    if ((int)g.size() > max_recvs) return 0;   // this protocol has no receive groups that large
  constexpr size_t SMALL = 1024, LARGE = 96 << 10;
  const int ns = (int)c.sends.size();
  if (g_rank == 0) {
    std::vector<std::vector<uint8_t>> buf(ns);
    std::vector<void*> mh(ns), req(ns, nullptr);
    for (int i = 0; i < ns; ++i) {
      buf[i].resize(c.sends[i].large ? LARGE : SMALL);
      fill(buf[i], 4000 + i);
      OK(net->regMr(p.s, buf[i].data(), buf[i].size(), NCCL_PTR_HOST, &mh[i]));
    }
    if (!late && barrier(sock)) FAIL("barrier");   // early: the receives are already posted
    std::deque<int> todo;
    for (int i = 0; i < ns; ++i) todo.push_back(i);
    std::vector<bool> done(ns, false);
    const auto t0 = Clock::now();
    while (!todo.empty()) {
      std::set<int> held;
      for (size_t round = todo.size(); round > 0; --round) {
        const int i = todo.front();
        todo.pop_front();
        if (!held.count(c.sends[i].tag)) {
          OK(net->isend(p.s, buf[i].data(), buf[i].size(), c.sends[i].tag, mh[i], nullptr, &req[i]));
          if (req[i]) continue;
          held.insert(c.sends[i].tag);
        }
        todo.push_back(i);
      }
      for (int i = 0; i < ns; ++i) {   // keep accepted sends moving
        if (!req[i] || done[i]) continue;
        int d = 0;
        OK(net->test(req[i], &d, nullptr));
        done[i] = d != 0;
      }
      if (expired(t0)) FAIL("%s (%s): %zu sends were never accepted", c.name, late ? "late" : "early", todo.size());
    }
    for (bool pending = true; pending;) {
      pending = false;
      for (int i = 0; i < ns; ++i) {
        if (done[i]) continue;
        int d = 0;
        OK(net->test(req[i], &d, nullptr));
        done[i] = d != 0;
        pending = pending || !done[i];
      }
      if (expired(t0)) FAIL("%s (%s): sends did not complete", c.name, late ? "late" : "early");
    }
    for (int i = 0; i < ns; ++i) OK(net->deregMr(p.s, mh[i]));
  } else {
    if (late) usleep(30000);   // let the small sends leave eagerly first
    const int ng = (int)c.groups.size();
    std::vector<std::vector<std::vector<uint8_t>>> buf(ng);
    std::vector<std::vector<void*>> mh(ng);
    std::vector<void*> req(ng, nullptr);
    std::map<int, int> seen;   // tag -> how many entries of it were posted so far
    std::vector<std::vector<int>> source(ng);   // which send each entry must receive
    for (int g = 0; g < ng; ++g) {
      const int n = (int)c.groups[g].size();
      buf[g].resize(n);
      mh[g].resize(n);
      void* data[8];
      size_t sizes[8];
      int tags[8];
      for (int k = 0; k < n; ++k) {
        const int tag = c.groups[g][k];
        int nth = seen[tag]++, src = -1;
        for (int i = 0; i < ns && src < 0; ++i)
          if (c.sends[i].tag == tag && nth-- == 0) src = i;
        if (src < 0) FAIL("%s: the table posts more receives of tag %d than sends", c.name, tag);
        source[g].push_back(src);
        buf[g][k].assign(LARGE + 64, 0);
        data[k] = buf[g][k].data();
        sizes[k] = buf[g][k].size();
        tags[k] = tag;
        OK(net->regMr(p.r, data[k], sizes[k], NCCL_PTR_HOST, &mh[g][k]));
      }
      if (post_recv(p.r, n, data, sizes, tags, mh[g].data(), &req[g])) return 1;
    }
    if (!late && barrier(sock)) FAIL("barrier");
    for (int g = 0; g < ng; ++g) {
      const int n = (int)c.groups[g].size();
      std::vector<void*> one{req[g]};
      std::vector<int> got;
      if (wait_all(one, &got, n)) FAIL("%s (%s): receive %d did not complete", c.name, late ? "late" : "early", g);
      for (int k = 0; k < n; ++k) {
        const int src = source[g][k];
        std::vector<uint8_t> want(c.sends[src].large ? LARGE : SMALL);
        fill(want, 4000 + src);
        if ((size_t)got[k] != want.size())
          FAIL("%s (%s): receive %d entry %d (tag %d) reports %d bytes, send %d has %zu", c.name, late ? "late" : "early", g, k,
               c.groups[g][k], got[k], src, want.size());
        if (memcmp(want.data(), buf[g][k].data(), want.size()))
          FAIL("%s (%s): receive %d entry %d (tag %d) does not hold send %d", c.name, late ? "late" : "early", g, k,
               c.groups[g][k], src);
        OK(net->deregMr(p.r, mh[g][k]));
      }
    }
  }
  if (barrier(sock)) FAIL("barrier");
  return 0;
}

static int scenario_eager_multirecv(int sock) {
  ncclNetProperties_v11_t props;
  memset(&props, 0, sizeof(props));
  OK(net->getProperties(0, &props));
  Pair p;
  if (connect_pair(0, sock, &p)) return 1;
  const bool S = false, L = true;
  auto two_groups_of_8 = [](const char* name, const std::vector<int>& tag_order, bool large) {
    EmrCase c;
    c.name = name;
    for (int tag : tag_order) c.sends.push_back({tag, large});
    c.groups = {{0, 1, 2, 3, 4, 5, 6, 7}, {0, 1, 2, 3, 4, 5, 6, 7}};
    return c;
  };
  // tag 1 of the second group is sent before tag 7 of the first
  const std::vector<int> cuts_in = {0, 1, 2, 3, 4, 5, 6, 1, 7, 0, 2, 3, 4, 5, 6, 7};
  const std::vector<int> alternating = {0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7};
  std::vector<EmrCase> cases = {
      {"one small send, one receive", {{1, S}}, {{1}}},
      {"four small sends, four receives", {{1, S}, {1, S}, {1, S}, {1, S}}, {{1}, {1}, {1}, {1}}},
      {"group of two, both eager", {{20, S}, {21, S}}, {{20, 21}}},
      {"group of three, eager and write mixed", {{10, S}, {11, L}, {12, S}}, {{10, 11, 12}}},
      {"group of two, both large", {{30, L}, {31, L}}, {{30, 31}}},
      {"eager across a single receive and a group", {{1, S}, {40, S}, {41, S}}, {{1}, {40, 41}}},
      {"eager sends in the order of two groups' tags", {{51, S}, {53, S}, {50, S}, {52, S}}, {{51, 53}, {50, 52}}},
      {"eager sends across the order of two groups' tags", {{50, S}, {51, S}, {52, S}, {53, S}}, {{51, 53}, {50, 52}}},
      {"two groups of four, every eager/write pairing per tag",
       {{60, S}, {61, S}, {62, L}, {63, L}, {60, S}, {61, L}, {62, S}, {63, L}},
       {{60, 61, 62, 63}, {60, 61, 62, 63}}},
      {"four groups with the same two tags",
       {{70, S}, {71, S}, {70, S}, {71, S}, {70, S}, {71, S}, {70, S}, {71, S}},
       {{70, 71}, {70, 71}, {70, 71}, {70, 71}}},
      two_groups_of_8("second group cuts in before the first is complete, all writes", cuts_in, L),
      two_groups_of_8("second group cuts in before the first is complete, all eager", cuts_in, S),
      {"second group cuts in, eager and write mixed",
       {{0, S}, {1, S}, {2, L}, {1, S}, {3, L}, {0, S}, {2, L}, {3, L}},
       {{0, 1, 2, 3}, {0, 1, 2, 3}}},
      {"three groups interleaved, eager / large / eager",
       {{0, S}, {1, S}, {0, L}, {0, S}, {1, L}, {1, S}},
       {{0, 1}, {0, 1}, {0, 1}}},
      two_groups_of_8("two groups of eight alternating send by send, all writes", alternating, L),
      two_groups_of_8("two groups of eight alternating send by send, all eager", alternating, S),
      {"eager batch spanning three groups of four",
       {{1, S}, {2, S}, {3, S}, {4, S}, {10, S}, {11, S}, {12, S}, {13, S}, {20, S}, {21, S}, {22, S}, {23, S}},
       {{1, 2, 3, 4}, {10, 11, 12, 13}, {20, 21, 22, 23}}},
      {"eager batch across single, group, single, group",
       {{1, S}, {50, S}, {51, S}, {1, S}, {60, S}, {61, S}},
       {{1}, {50, 51}, {1}, {60, 61}}},
      {"an eager send that belongs to a later receive than the large sends behind it",
       {{30, S}, {40, S}, {31, L}, {20, L}},
       {{30, 31}, {20}, {40}}},
      {"eager sends for the third group while the first two take writes",
       {{5, S}, {6, S}, {1, L}, {2, L}, {3, L}, {4, L}},
       {{1, 2}, {3, 4}, {5, 6}}},
  };
  for (const EmrCase& c : cases)
    for (int late = 0; late < 2; ++late)
      if (run_emr_case(c, p, sock, late != 0, props.maxRecvs)) return 1;
  return close_pair(&p);
}

struct Scenario {
  const char* name;
  int (*fn)(int);
};
static const Scenario kScenarios[] = {
    {"connection", scenario_connection},     {"message_transfer", scenario_message_transfer},
    {"pingpong", scenario_pingpong},         {"grouped_recv", scenario_grouped_recv},
    {"eager", scenario_eager},               {"reuse_listen", scenario_reuse_listen},
    {"inflight_close", scenario_inflight_close}, {"threads", scenario_threads},
    {"bandwidth", scenario_bandwidth},       {"proxy_pattern", scenario_proxy_pattern},
    {"device_transfer", scenario_device_transfer}, {"eager_multirecv", scenario_eager_multirecv},
    {"device_bandwidth", scenario_device_bandwidth}, {"seq_wrap", scenario_seq_wrap},
    {"dmabuf_registration", scenario_dmabuf_registration}, {"test_call_cost", scenario_test_call_cost},
};

static int run_rank(const char* so, const char* only, int sock) {
  g_sock = sock;
  void* h = dlopen(so, RTLD_NOW | RTLD_LOCAL);
  if (!h) FAIL("dlopen(%s): %s", so, dlerror());
  net = (ncclNet_v11_t*)dlsym(h, "ncclNetPlugin_v11");
  if (!net) FAIL("ncclNetPlugin_v11 not exported");
  OK(net->init(&g_ctx, 0x1234, nullptr, logger, nullptr));
  int rc = 0;
  if (only) {
    bool known = false;
    for (const auto& s : kScenarios) known = known || !strcmp(only, s.name);
    if (!known) FAIL("no scenario called %s", only);
  }
  for (const auto& s : kScenarios) {
    if (only && strcmp(only, s.name)) continue;
    const int r = s.fn(sock);
    fprintf(stderr, "[rank %d] %-18s %s\n", g_rank, s.name, r ? "FAILED" : "ok");
    if (r) {
      rc = 1;
      break;  // the peer will time out on its side; do not continue out of step
    }
  }
  if (!rc) OK(net->finalize(g_ctx));
  return rc;
}

int main(int argc, char** argv) {
  const char* so = argc > 1 ? argv[1] : "./libnccl-net-ofi-b200.so";
  const char* only = argc > 2 ? argv[2] : nullptr;
  int sv[2];
  if (socketpair(AF_UNIX, SOCK_STREAM, 0, sv) != 0) return 2;
  const pid_t pid = fork();
  if (pid < 0) return 2;
  if (pid == 0) {
    close(sv[0]);
    g_rank = 1;
    _exit(run_rank(so, only, sv[1]));
  }
  close(sv[1]);
  g_rank = 0;
  const int rc0 = run_rank(so, only, sv[0]);
  close(sv[0]);  // a peer blocked in a barrier sees end-of-file instead of waiting forever
  int status = 0;
  waitpid(pid, &status, 0);
  const int rc1 = WIFEXITED(status) ? WEXITSTATUS(status) : 3;
  if (rc0 || rc1) {
    fprintf(stderr, "FAILED: rank0=%d rank1=%d\n", rc0, rc1);
    return 1;
  }
  printf("ok\n");
  return 0;
}
