// GPU test of the plugin's own kernels (copy with completion flag, eager pack) through the driver
// shim: byte-exact against host memcpy for aligned and unaligned addresses, odd sizes, slot reuse
// past the pool size. Exit status 0 = pass, 77 = no GPU here.
#include <algorithm>
#include <chrono>
#include <functional>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "b200net/cuda_shim.h"
#include "b200net/net_kernels.h"
#include "test_util.h"

using namespace b200net;

static bool wait_until(const std::function<bool()>& f, double seconds) {
  const auto t0 = std::chrono::steady_clock::now();
  while (!f()) {
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > seconds) return false;
  }
  return true;
}

int main() {
  // no rescue by age in this test: a queued transfer has to leave because the launches before it are
  // seen complete, or it stays queued for longer than any wait below
  setenv("B200NET_COPY_BATCH_MAX_AGE_US", "5000000", 1);
  if (cuda::init() != 0 || cuda::device_count() < 1) {
    printf("no GPU: skipped\n");
    return 77;
  }
  CHECK_EQ(cuda::ensure_primary_ctx(0), 0);
  NetKernels* nk = NetKernels::get();
  CHECK(nk != nullptr);
  if (!nk) TEST_MAIN_END();
  cuda::Stream st = nullptr;
  CHECK_EQ(cuda::stream_create(&st), 0);
  const size_t cap = (64u << 20) + 4096;
  void *dsrc = nullptr, *ddst = nullptr;
  CHECK_EQ(cuda::mem_alloc(&dsrc, cap), 0);
  CHECK_EQ(cuda::mem_alloc(&ddst, cap), 0);
  std::vector<uint8_t> host(cap), back(cap);
  std::mt19937_64 rng(0);
  for (size_t i = 0; i < cap; i += 8) {
    const uint64_t v = rng();
    memcpy(&host[i], &v, std::min<size_t>(8, cap - i));
  }
  CHECK_EQ(cuda::memcpy_async(dsrc, host.data(), cap, st), 0);
  CHECK_EQ(cuda::stream_synchronize(st), 0);

  // ---- copy with completion flag
  struct Case { size_t n, src_off, dst_off; int ctas; };
  const Case cases[] = {{8, 0, 0, 0},       {1, 3, 5, 0},          {4096, 0, 0, 1},        {4099, 16, 32, 0},
                        {65536, 1, 0, 0},   {(1u << 20) + 7, 0, 0, 0}, {(16u << 20), 16, 16, 0}, {(64u << 20), 0, 0, 32},
                        {12345, 7, 7, 3},
                        // 16-byte aligned stripes of 64 KiB and more: the bulk-copy kernel (one piece, a ragged
                        // last piece, more CTAs than pieces, many pieces per CTA)
                        {65536, 0, 0, 0},   {65536 + 16, 16, 48, 0}, {(1u << 20) + 16, 0, 32, 5}, {(3u << 20) + 48, 64, 16, 0},
                        {32768 * 3, 0, 0, 16}, {(48u << 20), 0, 0, 2}};
  for (const Case& c : cases) {
    // poison the destination so stale bytes cannot pass
    std::vector<uint8_t> poison(c.n + 64, 0xA5);
    CHECK_EQ(cuda::memcpy_async(static_cast<char*>(ddst) + c.dst_off, poison.data(), c.n + 32, st), 0);
    int slot = -1;
    CHECK_EQ(nk->copy_flag(static_cast<char*>(ddst) + c.dst_off, static_cast<char*>(dsrc) + c.src_off, c.n, st, c.ctas, &slot), 0);
    CHECK(wait_until([&] { return nk->done(slot); }, 10.0));
    nk->release(slot);
    CHECK_EQ(cuda::memcpy_async(back.data(), static_cast<char*>(ddst) + c.dst_off, c.n + 32, st), 0);
    CHECK_EQ(cuda::stream_synchronize(st), 0);
    CHECK(memcmp(back.data(), host.data() + c.src_off, c.n) == 0);
    bool tail_intact = true;
    for (size_t i = c.n; i < c.n + 32; ++i) tail_intact &= back[i] == 0xA5;
    CHECK(tail_intact);   // nothing written past the end
  }
  // slots are recycled: more transfers than the pool has slots, several in flight at once
  for (int round = 0; round < 3 * NetKernels::NUM_FLAGS / 8; ++round) {
    int slots[8];
    for (int j = 0; j < 8; ++j)
      CHECK_EQ(nk->copy_flag(static_cast<char*>(ddst) + j * 4096, static_cast<char*>(dsrc) + (round % 5) * 512 + j * 4096, 4096,
                             st, 1, &slots[j]), 0);
    for (int j = 0; j < 8; ++j) {
      CHECK(wait_until([&] { return nk->done(slots[j]); }, 10.0));
      nk->release(slots[j]);
    }
  }
  CHECK_EQ(cuda::memcpy_async(back.data(), ddst, 8 * 4096, st), 0);
  CHECK_EQ(cuda::stream_synchronize(st), 0);
  const int last_round = 3 * NetKernels::NUM_FLAGS / 8 - 1;
  CHECK(memcmp(back.data(), host.data() + (last_round % 5) * 512, 8 * 4096) == 0);

  // ---- queued copies: bursts leave in launches of the batch kernel, every transfer with its own
  // completion word. The regions do not overlap; sizes and offsets mix the bulk path (16-byte
  // aligned, 64 KiB and more), the vector path, unaligned ends and an empty transfer.
  {
    struct Q { size_t n, src_off, dst_off; };
    const Q qs[] = {{2u << 20, 0, 0},          {65536, 16, 32},          {100, 3, 1},           {0, 0, 0},
                    {(1u << 20) + 5, 7, 9},    {3u << 20, 64, 128},      {4096, 0, 0},          {65536 + 16, 0, 16},
                    {12345, 1, 2},             {8u << 20, 0, 0},         {1u << 20, 48, 16},    {70000, 5, 5},
                    {16, 0, 0},                {1u << 20, 0, 0},         {262144, 16, 16},      {1, 0, 0},
                    {2u << 20, 32, 0},         {65536, 0, 0},            {999, 0, 3},           {4u << 20, 0, 16}};
    const int nq = static_cast<int>(sizeof(qs) / sizeof(qs[0]));
    const size_t region = 9u << 20;   // per transfer; nq regions do not fit the buffers at once: two passes
    const uint64_t batches_before = nk->batch_launches(), jobs_before = nk->batched_jobs();
    for (int pass = 0; pass < 3; ++pass) {
      const int per_pass = 7;   // 7 regions of 9 MiB fit the 64 MiB buffers
      for (int base = 0; base < nq; base += per_pass) {
        const int cnt = std::min(per_pass, nq - base);
        std::vector<uint8_t> poison(region, 0x5A);
        for (int i = 0; i < cnt; ++i) CHECK_EQ(cuda::memcpy_async(static_cast<char*>(ddst) + i * region, poison.data(), region, st), 0);
        CHECK_EQ(cuda::stream_synchronize(st), 0);
        int slots[per_pass];
        for (int i = 0; i < cnt; ++i) {
          const Q& q = qs[base + i];
          CHECK_EQ(nk->copy_queue(static_cast<char*>(ddst) + i * region + q.dst_off, static_cast<char*>(dsrc) + i * region + q.src_off,
                                  q.n, &slots[i]), 0);
        }
        for (int i = 0; i < cnt; ++i) {
          CHECK(wait_until([&] { return nk->status(slots[i]) != 0; }, 10.0));
          CHECK_EQ(nk->status(slots[i]), 1);
          nk->release(slots[i]);
        }
        CHECK_EQ(cuda::memcpy_async(back.data(), ddst, cnt * region, st), 0);
        CHECK_EQ(cuda::stream_synchronize(st), 0);
        for (int i = 0; i < cnt; ++i) {
          const Q& q = qs[base + i];
          const uint8_t* got = back.data() + i * region;
          CHECK(memcmp(got + q.dst_off, host.data() + i * region + q.src_off, q.n) == 0);
          bool around = true;
          for (size_t b = 0; b < q.dst_off; ++b) around &= got[b] == 0x5A;
          for (size_t b = q.dst_off + q.n; b < q.dst_off + q.n + 64; ++b) around &= got[b] == 0x5A;
          CHECK(around);   // nothing written before the start or past the end
        }
      }
    }
    // with seven transfers queued back to back some of them must have shared a launch
    CHECK(nk->batch_launches() > batches_before);
    CHECK(nk->batched_jobs() - jobs_before >= 2 * (nk->batch_launches() - batches_before));
    // finished transfers whose slots are still held do not count as launches in flight: NCCL tests
    // the requests of a channel in order, so a finished one can stay unreleased for long
    {
      int first[6], later = -1;
      for (int& f : first) {
        CHECK_EQ(nk->copy_queue(static_cast<char*>(ddst) + (2u << 20), dsrc, 4096, &f), 0);
        CHECK(wait_until([&] { return nk->status(f) != 0; }, 10.0));   // each one a launch of its own
      }
      CHECK_EQ(nk->copy_queue(static_cast<char*>(ddst) + (3u << 20), dsrc, 4096, &later), 0);
      CHECK(wait_until([&] { return nk->status(later) != 0; }, 3.0));
      CHECK_EQ(nk->status(later), 1);
      for (int f : first) nk->release(f);
      nk->release(later);
    }
    // a slot given back before its launch never runs: the destination keeps its bytes
    std::vector<uint8_t> mark(4096, 0x77);
    CHECK_EQ(cuda::memcpy_async(ddst, mark.data(), 4096, st), 0);
    CHECK_EQ(cuda::stream_synchronize(st), 0);
    int held[4], dropped = -1;
    for (int& h : held) CHECK_EQ(nk->copy_queue(static_cast<char*>(ddst) + (1u << 20), dsrc, 1u << 20, &h), 0);   // keeps launches in flight
    CHECK_EQ(nk->copy_queue(ddst, static_cast<char*>(dsrc) + 4096, 4096, &dropped), 0);
    nk->release(dropped);
    for (int h : held) {
      CHECK(wait_until([&] { return nk->status(h) != 0; }, 10.0));
      nk->release(h);
    }
    nk->poll();
    CHECK_EQ(cuda::stream_synchronize(nk->stream()), 0);
    CHECK_EQ(cuda::memcpy_async(back.data(), ddst, 4096, st), 0);
    CHECK_EQ(cuda::stream_synchronize(st), 0);
    // (when the queue happened to be empty at that moment the transfer was launched at once and did
    // run: both outcomes leave whole bytes, never a torn mix)
    CHECK(memcmp(back.data(), mark.data(), 4096) == 0 || memcmp(back.data(), host.data() + 4096, 4096) == 0);
  }

  // ---- eager pack: header, payload and flag in one pinned slot
  const size_t sizes[] = {1, 7, 8, 15, 16, 17, 255, 1024, 4097, 8191, 8192};
  for (int rep = 0; rep < 2 * NetKernels::NUM_EAGER_SLOTS / 11 + 2; ++rep) {
    for (size_t n : sizes) {
      const size_t off = (rep * 13 + n) % 64;   // aligned and unaligned sources
      int slot = -1;
      CHECK_EQ(nk->eager_pack(static_cast<char*>(dsrc) + off, n, 0x1111000000000000ull + rep, n, st, &slot), 0);
      CHECK(wait_until([&] { return nk->eager_done(slot); }, 10.0));
      const uint8_t* s = nk->eager_slot(slot);
      uint64_t h0, h1;
      memcpy(&h0, s, 8);
      memcpy(&h1, s + 8, 8);
      CHECK_EQ(h0, 0x1111000000000000ull + rep);
      CHECK_EQ(h1, n);
      CHECK(memcmp(s + 16, host.data() + off, n) == 0);
      nk->eager_release(slot);
    }
  }
  int slot = -1;
  CHECK_EQ(nk->eager_pack(dsrc, NetKernels::EAGER_PAYLOAD_MAX + 1, 0, 0, st, &slot), -EMSGSIZE);
  CHECK(nk->launches() > 0);
  cuda::mem_free(dsrc);
  cuda::mem_free(ddst);
  cuda::stream_destroy(st);
  TEST_MAIN_END();
}
