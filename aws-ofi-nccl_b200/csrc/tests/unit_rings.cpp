// dlist, spinlock, SPSC ring, MPSC ring (wrap-around, full/empty, concurrent producers), ep_addr_list.
#include <atomic>
#include <thread>
#include <vector>
#include "b200net/dlist.h"
#include "b200net/ep_addr_list.h"
#include "b200net/mpsc_ring.h"
#include "b200net/spinlock.h"
#include "b200net/spsc_ring.h"
#include "test_util.h"
using namespace b200net;

struct Item { int v; DListNode node; };

int main() {
  {  // dlist
    DList l; Item it[5];
    CHECK(l.empty());
    for (int i = 0; i < 5; ++i) { it[i].v = i; l.push_back(&it[i].node); }
    CHECK_EQ(l.size(), 5u);
    DList::remove(&it[2].node);
    l.push_front(&it[2].node);
    int order[5], n = 0;
    l.for_each_safe([&](DListNode* nd) { order[n++] = B200NET_CONTAINER_OF(nd, Item, node)->v; if (order[n - 1] == 3) DList::remove(nd); });
    int want[5] = {2, 0, 1, 3, 4};
    for (int i = 0; i < 5; ++i) CHECK_EQ(order[i], want[i]);
    CHECK_EQ(l.size(), 4u);
    CHECK_EQ(B200NET_CONTAINER_OF(l.pop_front(), Item, node)->v, 2);
    while (l.pop_front()) {}
    CHECK(l.empty() && l.front() == nullptr);
  }
  {  // spinlock protects a counter
    Spinlock sl; long counter = 0;
    std::vector<std::thread> th;
    for (int t = 0; t < 4; ++t) th.emplace_back([&] { for (int i = 0; i < 50000; ++i) { sl.lock(); ++counter; sl.unlock(); } });
    for (auto& t : th) t.join();
    CHECK_EQ(counter, 200000);
    CHECK(sl.try_lock()); CHECK(!sl.try_lock()); sl.unlock();
  }
  {  // SPSC: capacity-1 usable, FIFO across wrap
    SpscRing<int> r(8);
    CHECK_EQ(r.usable(), 7u);
    int out;
    CHECK(!r.pop(out));
    for (int round = 0; round < 5; ++round) {
      for (int i = 0; i < 7; ++i) CHECK(r.push(round * 10 + i));
      CHECK(!r.push(99));
      for (int i = 0; i < 7; ++i) { CHECK(r.pop(out)); CHECK_EQ(out, round * 10 + i); }
      CHECK(r.empty());
    }
    std::thread prod([&] { for (int i = 0; i < 100000;) if (r.push(i)) ++i; });
    for (int i = 0; i < 100000;) if (r.pop(out)) { CHECK_EQ(out, i); ++i; }
    prod.join();
  }
  {  // MPSC: all slots usable, full/empty, wrap, multi-producer
    MpscRing<uint64_t> r(8);
    CHECK_EQ(r.capacity(), 8u);
    uint64_t out;
    CHECK(!r.pop(out));
    for (int round = 0; round < 5; ++round) {
      for (uint64_t i = 0; i < 8; ++i) CHECK(r.push(round * 100 + i));
      CHECK(!r.push(7));
      for (uint64_t i = 0; i < 8; ++i) { CHECK(r.pop(out)); CHECK_EQ(out, round * 100 + i); }
      CHECK(r.empty());
    }
    MpscRing<uint64_t> big(1024);
    const int P = 4, N = 50000;
    std::vector<std::thread> th;
    for (int p = 0; p < P; ++p) th.emplace_back([&, p] { for (int i = 0; i < N;) if (big.push((uint64_t(p) << 32) | i)) ++i; });
    std::vector<int> next(P, 0);
    for (int got = 0; got < P * N;) {
      if (big.pop(out)) { const int p = out >> 32; CHECK_EQ(static_cast<int>(out & 0xffffffff), next[p]); ++next[p]; ++got; }
    }
    for (auto& t : th) t.join();
    // byte ring: gather of two fragments, oversize rejected, peek/release
    alignas(64) static char mem[4096];
    CHECK(MpscByteRing::footprint(4, 48) <= sizeof(mem));
    MpscByteRing br = MpscByteRing::create(mem, 4, 48);
    CHECK(!br.push(mem, 49));
    CHECK(br.push("abcd", 4, "efgh", 4));
    size_t len; const void* p = br.peek(&len);
    CHECK(p && len == 8 && memcmp(p, "abcdefgh", 8) == 0);
    br.release_front();
    CHECK(br.peek(&len) == nullptr);
    MpscByteRing again = MpscByteRing::attach(mem);  // a second mapping of the same storage
    CHECK(again.push("x", 1)); CHECK(!br.empty());
  }
  {  // ep_addr_list
    EpAddrList l; int e1, e2;
    CHECK(l.get("A") == nullptr);
    CHECK_EQ(l.insert(&e1, "A"), 0);
    CHECK_EQ(l.insert(&e1, "B"), -EINVAL);
    CHECK(l.get("A") == nullptr);       // e1 already talks to A
    CHECK(l.get("B") == &e1);           // now paired with B too
    CHECK(l.get("B") == nullptr);
    CHECK_EQ(l.insert(&e2, "B"), 0);
    CHECK(l.get("A") == &e2);
    CHECK_EQ(l.remove(&e1), 0); CHECK_EQ(l.remove(&e1), -ENOENT);
    CHECK_EQ(l.size(), 1u);
  }
  TEST_MAIN_END();
}
