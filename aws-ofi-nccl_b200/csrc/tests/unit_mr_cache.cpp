// MR cache: containment lookups, page rounding, refcounts, EEXIST, dmabuf keys, endpoint scoping.
#include <cerrno>
#include "b200net/mr_cache.h"
#include "test_util.h"
using namespace b200net;
int main() {
  MrCache c(4, 4096);
  char* base = reinterpret_cast<char*>(0x100000);
  int h1, h2, h3;
  CHECK(c.lookup(MrCacheKey::from_iovec(base, 100)) == nullptr);
  CHECK_EQ(c.misses(), 1u);
  CHECK_EQ(c.insert(MrCacheKey::from_iovec(base + 10, 8000), &h1), 0);       // pages [0x100000, 0x102000)
  CHECK_EQ(c.insert(MrCacheKey::from_iovec(base, 8192), &h2), -EEXIST);      // same page range
  CHECK(c.lookup(MrCacheKey::from_iovec(base + 4096, 4096)) == &h1);         // contained
  CHECK(c.lookup(MrCacheKey::from_iovec(base + 8000, 500)) == nullptr);      // crosses the end
  CHECK(c.lookup(MrCacheKey::from_iovec(base - 1, 2)) == nullptr);           // starts before
  CHECK_EQ(c.hits(), 1u);
  CHECK_EQ(c.insert(MrCacheKey::from_iovec(base + 0x10000, 4096), &h2), 0);
  CHECK_EQ(c.insert(MrCacheKey::from_iovec(base - 0x10000, 4096), &h3), 0);  // keeps the vector sorted
  CHECK_EQ(c.size(), 3u);
  CHECK(c.lookup(MrCacheKey::from_iovec(base - 0x10000 + 5, 10)) == &h3);
  // refcounts: h1 has 2 refs (insert + lookup)
  CHECK_EQ(c.del(&h1), 0);
  CHECK_EQ(c.del(&h1), 1);
  CHECK_EQ(c.del(&h1), -ENOENT);
  CHECK(c.lookup(MrCacheKey::from_iovec(base + 4096, 16)) == nullptr);
  // page_range arithmetic
  uintptr_t b; size_t pages;
  c.page_range(MrCacheKey::from_iovec(base + 4095, 2), &b, &pages);
  CHECK_EQ(b, 0x100000u); CHECK_EQ(pages, 2u);
  c.page_range(MrCacheKey::from_iovec(base, 0), &b, &pages);
  CHECK_EQ(pages, 1u);
  // dmabuf keys only match the same fd; endpoint-scoped keys only the same endpoint
  int h4, h5, ep1, ep2;
  CHECK_EQ(c.insert(MrCacheKey::from_dmabuf(7, 0, base + 0x40000, 4096), &h4), 0);
  CHECK(c.lookup(MrCacheKey::from_dmabuf(8, 0, base + 0x40000, 64)) == nullptr);
  CHECK(c.lookup(MrCacheKey::from_iovec(base + 0x40000, 64)) == nullptr);
  CHECK(c.lookup(MrCacheKey::from_dmabuf(7, 0, base + 0x40000, 64)) == &h4);
  CHECK_EQ(c.insert(MrCacheKey::from_iovec(base + 0x80000, 4096, &ep1), &h5), 0);
  CHECK(c.lookup(MrCacheKey::from_iovec(base + 0x80000, 8, &ep2)) == nullptr);
  CHECK(c.lookup(MrCacheKey::from_iovec(base + 0x80000, 8, &ep1)) == &h5);
  // exact keys (one device allocation each): two small allocations in one page never share a handle
  int a1, a2;
  CHECK_EQ(c.insert(MrCacheKey::from_allocation(base + 0x200000, 65), &a1), 0);
  CHECK(c.lookup(MrCacheKey::from_allocation(base + 0x200000 + 512, 72)) == nullptr);   // a neighbour in the same page
  CHECK_EQ(c.insert(MrCacheKey::from_allocation(base + 0x200000 + 512, 72), &a2), 0);
  CHECK(c.lookup(MrCacheKey::from_allocation(base + 0x200000, 65)) == &a1);
  CHECK(c.lookup(MrCacheKey::from_allocation(base + 0x200000 + 512, 72)) == &a2);
  CHECK(c.lookup(MrCacheKey::from_allocation(base + 0x200000, 64)) == nullptr);         // same base, other size
  CHECK(c.lookup(MrCacheKey::from_iovec(base + 0x200000, 16)) == nullptr);              // a containment key never hits an exact entry
  CHECK_EQ(c.insert(MrCacheKey::from_allocation(base + 0x200000, 65), &a2), -EEXIST);
  CHECK_EQ(c.del(&a1), 0);
  CHECK_EQ(c.del(&a1), 1);
  TEST_MAIN_END();
}
