#include "b200net/scheduler.h"

#include <new>

#include "b200net/assert.h"
#include "b200net/math.h"

namespace b200net {

static Freelist::Options schedule_pool_options() {
  Freelist::Options o;
  o.entry_size = sizeof(Schedule);
  o.initial_count = 16;
  o.grow_count = 16;
  o.entry_align = alignof(Schedule);
  o.name = "schedule pool";
  return o;
}

ThresholdScheduler::ThresholdScheduler(int num_rails, size_t min_stripe_size, size_t max_small_msg_size)
    : num_rails_(num_rails), min_stripe_(min_stripe_size), max_small_(max_small_msg_size),
      pool_(schedule_pool_options()) {
  B200NET_ASSERT_ALWAYS(num_rails >= 1 && num_rails <= MAX_NUM_RAILS);
  B200NET_ASSERT_ALWAYS(min_stripe_size > 0);
}

ThresholdScheduler::~ThresholdScheduler() = default;

// As many stripes as the message has min-stripe-sized pieces, capped by the rail count and then
// lowered to the largest divisor of the rail count, so that consecutive messages rotate evenly.
int ThresholdScheduler::num_stripes_for(size_t size, int num_rails, size_t min_stripe) {
  size_t n = clamp_to<size_t>(div_ceil<size_t>(size, min_stripe), 1, static_cast<size_t>(num_rails));
  while (num_rails % static_cast<int>(n) != 0) --n;
  return static_cast<int>(n);
}

size_t ThresholdScheduler::stripe_size_for(size_t size, int num_stripes) {
  return round_up<size_t>(div_ceil<size_t>(size, static_cast<size_t>(num_stripes)), STRIPE_ALIGN);
}

Schedule* ThresholdScheduler::get_schedule(size_t size, int num_rails) {
  B200NET_ASSERT_ALWAYS(num_rails >= 1 && num_rails <= MAX_NUM_RAILS);
  ScopedLock g(mu_);
  FreelistEntry* fe = pool_.entry_alloc();
  if (!fe) return nullptr;
  Schedule* s = new (fe->ptr) Schedule();
  s->fl_entry = fe;
  if (size < max_small_ || num_rails == 1) {
    // latency path: one rail, chosen round-robin
    s->num_xfer_infos = 1;
    s->xfers[0] = XferInfo{static_cast<int>(rr_counter_ % static_cast<unsigned>(num_rails)), 0, size};
    rr_counter_ = (rr_counter_ + 1) % static_cast<unsigned>(num_rails);
    return s;
  }
  const int n = num_stripes_for(size, num_rails, min_stripe_);
  const size_t stripe = stripe_size_for(size, n);
  size_t left = size, off = 0;
  int used = 0;
  for (int i = 0; i < n && left > 0; ++i) {
    const size_t len = left < stripe ? left : stripe;
    s->xfers[used++] = XferInfo{static_cast<int>((rr_counter_ + static_cast<unsigned>(i)) % static_cast<unsigned>(num_rails)), off, len};
    off += len;
    left -= len;
  }
  s->num_xfer_infos = static_cast<size_t>(used);
  rr_counter_ = (rr_counter_ + static_cast<unsigned>(n)) % static_cast<unsigned>(num_rails);
  return s;
}

void ThresholdScheduler::release_schedule(Schedule* s) {
  if (!s) return;
  ScopedLock g(mu_);
  FreelistEntry* fe = s->fl_entry;
  s->~Schedule();
  pool_.entry_free(fe);
}

}  // namespace b200net
