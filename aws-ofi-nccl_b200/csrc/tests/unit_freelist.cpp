// Freelist: growth up to the maximum, init/fini callbacks, registration callbacks seeing whole
// pages, entry alignment, and the leak path at destruction.
#include <set>
#include <vector>
#include "b200net/freelist.h"
#include "b200net/math.h"
#include "test_util.h"
using namespace b200net;

int main() {
  {  // simple: unbounded growth, distinct aligned entries
    Freelist::Options o;
    o.entry_size = 100; o.initial_count = 4; o.grow_count = 4; o.entry_align = 64;
    Freelist fl(o);
    std::set<void*> seen;
    std::vector<FreelistEntry*> es;
    for (int i = 0; i < 300; ++i) {
      FreelistEntry* e = fl.entry_alloc();
      CHECK(e != nullptr);
      CHECK(is_ptr_aligned(e->ptr, 64));
      CHECK(seen.insert(e->ptr).second);
      static_cast<char*>(e->ptr)[0] = 1; static_cast<char*>(e->ptr)[99] = 2;
      es.push_back(e);
    }
    CHECK(fl.block_count() > 1);
    for (auto* e : es) fl.entry_free(e);
    CHECK_EQ(fl.in_use(), 0u);
  }
  {  // bounded: allocation fails at max_count
    Freelist::Options o;
    o.entry_size = 1024; o.initial_count = 8; o.grow_count = 8; o.max_count = 16;
    Freelist fl(o);
    std::vector<FreelistEntry*> es;
    for (int i = 0; i < 16; ++i) { auto* e = fl.entry_alloc(); CHECK(e); es.push_back(e); }
    CHECK(fl.entry_alloc() == nullptr);
    fl.entry_free(es.back()); es.pop_back();
    CHECK(fl.entry_alloc() != nullptr);
    CHECK_EQ(fl.allocated(), 16u);
    for (auto* e : es) fl.entry_free(e);
    // one entry is deliberately left out: the destructor must report it
  }
  CHECK_EQ(Freelist::leaked_entries_total(), 1u);
  {  // registration callbacks: whole pages, handle propagated to entries, dereg per block
    int regs = 0, deregs = 0, inits = 0, finis = 0;
    {
      Freelist::Options o;
      o.entry_size = 8192 + 8; o.initial_count = 2; o.grow_count = 2; o.page_size = 4096;
      o.reg = [&](void* base, size_t bytes, void** h) {
        CHECK(is_ptr_aligned(base, 4096)); CHECK_EQ(bytes % 4096, 0u);
        *h = reinterpret_cast<void*>(static_cast<uintptr_t>(0x1000 + regs)); ++regs; return 0; };
      o.dereg = [&](void* h) { CHECK(h != nullptr); ++deregs; return 0; };
      o.entry_init = [&](void*) { ++inits; return 0; };
      o.entry_fini = [&](void*) { ++finis; };
      Freelist fl(o);
      std::vector<FreelistEntry*> es;
      for (int i = 0; i < 7; ++i) { auto* e = fl.entry_alloc(); CHECK(e && e->mr_handle != nullptr); es.push_back(e); }
      CHECK(regs >= 2);
      CHECK_EQ(static_cast<size_t>(regs), fl.block_count());
      for (auto* e : es) fl.entry_free(e);
    }
    CHECK_EQ(regs, deregs);
    CHECK_EQ(inits, finis);
    CHECK(inits >= 7);
  }
  {  // failing registration: allocation fails cleanly
    Freelist::Options o;
    o.entry_size = 64; o.initial_count = 0; o.grow_count = 4;
    o.reg = [](void*, size_t, void**) { return -1; };
    Freelist fl(o);
    CHECK(fl.entry_alloc() == nullptr);
    CHECK_EQ(fl.block_count(), 0u);
  }
  TEST_MAIN_END();
}
