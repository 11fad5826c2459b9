// Multi-rail scheduler: decides how one message is striped over the copy channels ("rails") of
// a connection. Small messages take a single rail chosen round-robin; larger ones are split into
// a number of stripes that divides the rail count, each stripe a multiple of 128 bytes
// (reference: src/nccl_ofi_scheduler.cpp, include/nccl_ofi_scheduler.h). On B200 a rail is an
// SM copy channel or a copy-engine stream towards the peer GPU instead of a NIC.
#pragma once
#include <cstddef>
#include <cstdint>
#include "b200net/pthread_wrap.h"
#include "b200net/freelist.h"

namespace b200net {

constexpr int MAX_NUM_RAILS = 8;
constexpr size_t STRIPE_ALIGN = 128;

struct XferInfo {
  int rail_id;
  size_t offset;
  size_t msg_size;
};

struct Schedule {
  size_t num_xfer_infos = 0;
  XferInfo xfers[MAX_NUM_RAILS];
  FreelistEntry* fl_entry = nullptr;  // owner bookkeeping
};

class ThresholdScheduler {
 public:
  ThresholdScheduler(int num_rails, size_t min_stripe_size = 128 * 1024, size_t max_small_msg_size = 64);
  ~ThresholdScheduler();
  // Returns a schedule from the pool (nullptr only if the pool cannot grow).
  Schedule* get_schedule(size_t size, int num_rails);
  void release_schedule(Schedule* s);
  int num_rails() const { return num_rails_; }
  size_t min_stripe_size() const { return min_stripe_; }
  // Pure functions exposed for tests and for the device-side striping of GIN puts.
  static int num_stripes_for(size_t size, int num_rails, size_t min_stripe);
  static size_t stripe_size_for(size_t size, int num_stripes);

 private:
  int num_rails_;
  size_t min_stripe_, max_small_;
  Mutex mu_;
  unsigned rr_counter_ TSA_GUARDED_BY(mu_) = 0;
  Freelist pool_ TSA_GUARDED_BY(mu_);
};

}  // namespace b200net
