// IdPool: lowest-free allocation, exhaustion, free/reuse, double free and range errors.
#include "b200net/idpool.h"
#include "test_util.h"
using namespace b200net;
int main() {
  for (size_t size : {1u, 63u, 64u, 65u, 200u}) {
    IdPool p(size);
    for (size_t i = 0; i < size; ++i) CHECK_EQ(p.allocate(), i);
    CHECK_EQ(p.allocate(), IdPool::ID_NONE);
    CHECK_EQ(p.in_use(), size);
    p.free_id(size / 2);
    CHECK_EQ(p.allocate(), size / 2);
    p.free_id(0);
    if (size > 3) { p.free_id(3); CHECK_EQ(p.allocate(), 0u); CHECK_EQ(p.allocate(), 3u); }
  }
  IdPool q(10);
  CHECK_THROWS(q.free_id(3));     // never allocated
  CHECK_THROWS(q.free_id(10));    // out of range
  uint64_t id = q.allocate();
  q.free_id(id);
  CHECK_THROWS(q.free_id(id));    // double free
  IdPool z(0);
  CHECK_EQ(z.allocate(), IdPool::ID_NONE);
  TEST_MAIN_END();
}
