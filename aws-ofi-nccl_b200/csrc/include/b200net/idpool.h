// Pool of small integer ids backed by a bit vector: allocate returns the lowest free id
// (ffsll over 64-bit words), or ID_NONE when exhausted; freeing an id that is not in use
// throws (reference: src/nccl_ofi_idpool.cpp).
#pragma once
#include <cstddef>
#include <cstdint>
#include "b200net/pthread_wrap.h"
#include <vector>

namespace b200net {

class IdPool {
 public:
  static constexpr uint64_t ID_NONE = ~uint64_t{0};
  explicit IdPool(size_t size);
  uint64_t allocate();          // lowest free id or ID_NONE
  void free_id(uint64_t id);    // throws std::logic_error on double free / out of range
  size_t size() const { return size_; }
  size_t in_use() const;

 private:
  size_t size_;
  mutable Mutex mu_;
  std::vector<uint64_t> free_bits_ TSA_GUARDED_BY(mu_);  // bit set = id free
};

}  // namespace b200net
