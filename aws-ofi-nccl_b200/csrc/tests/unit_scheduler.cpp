// Scheduler: exact {rail, offset, size} of every stripe against hand-computed schedules.
#include <vector>
#include "b200net/scheduler.h"
#include "test_util.h"
using namespace b200net;

struct Want { int rail; size_t off, len; };
static void expect(ThresholdScheduler& s, size_t size, int rails, std::vector<Want> want) {
  Schedule* sc = s.get_schedule(size, rails);
  CHECK(sc != nullptr);
  CHECK_EQ(sc->num_xfer_infos, want.size());
  for (size_t i = 0; i < want.size() && i < sc->num_xfer_infos; ++i) {
    CHECK_EQ(sc->xfers[i].rail_id, want[i].rail);
    CHECK_EQ(sc->xfers[i].offset, want[i].off);
    CHECK_EQ(sc->xfers[i].msg_size, want[i].len);
  }
  s.release_schedule(sc);
}

int main() {
  const size_t MS = 4096;  // min stripe
  {
    ThresholdScheduler s(4, MS, 64);
    // small messages: one rail, round robin 0,1,2,3,0
    for (int i = 0; i < 5; ++i) expect(s, 8, 4, {{i % 4, 0, 8}});
    expect(s, 0, 4, {{1, 0, 0}});  // zero-byte message still gets a rail
    // rr counter now at 2
    expect(s, 64, 4, {{2, 0, 64}});            // 64 is not "small" (< 64) but fits one stripe
    expect(s, MS, 4, {{3, 0, MS}});            // exactly one stripe
    expect(s, MS + 1, 4, {{0, 0, 2176}, {1, 2176, 1921}});  // 2 stripes: ceil(4097/2)=2049 -> 2176 (x128)
    expect(s, 3 * MS, 4, {{2, 0, 6144}, {3, 6144, 6144}});  // 3 pieces -> largest divisor of 4 below = 2
    expect(s, 4 * MS, 4, {{0, 0, MS}, {1, MS, MS}, {2, 2 * MS, MS}, {3, 3 * MS, MS}});
    expect(s, 100 * MS, 4, {{0, 0, 25 * MS}, {1, 25 * MS, 25 * MS}, {2, 50 * MS, 25 * MS}, {3, 75 * MS, 25 * MS}});
    // sizes that do not divide: last stripe is the remainder, every stripe start is 128-aligned
    Schedule* sc = s.get_schedule(4 * MS + 77, 4);
    size_t total = 0;
    for (size_t i = 0; i < sc->num_xfer_infos; ++i) { CHECK_EQ(sc->xfers[i].offset % 128, 0u); CHECK_EQ(sc->xfers[i].offset, total); total += sc->xfers[i].msg_size; }
    CHECK_EQ(total, 4 * MS + 77);
    s.release_schedule(sc);
  }
  {
    ThresholdScheduler s(3, MS, 64);
    expect(s, 2 * MS, 3, {{0, 0, 2 * MS}});   // 2 does not divide 3 -> 1 stripe
    expect(s, 3 * MS, 3, {{1, 0, MS}, {2, MS, MS}, {0, 2 * MS, MS}});
  }
  {
    ThresholdScheduler s(1, MS, 64);
    expect(s, 10 * MS, 1, {{0, 0, 10 * MS}});
  }
  CHECK_EQ(ThresholdScheduler::num_stripes_for(1 << 20, 8, 128 * 1024), 8);
  CHECK_EQ(ThresholdScheduler::num_stripes_for(5 * 128 * 1024, 8, 128 * 1024), 4);
  CHECK_EQ(ThresholdScheduler::stripe_size_for(1000, 3), 384u);
  CHECK_THROWS(ThresholdScheduler(0));
  CHECK_THROWS(ThresholdScheduler(MAX_NUM_RAILS + 1));
  TEST_MAIN_END();
}
