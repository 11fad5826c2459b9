#include "b200net/idpool.h"

#include <stdexcept>

#include "b200net/math.h"

namespace b200net {

IdPool::IdPool(size_t size) : size_(size), free_bits_(div_ceil<size_t>(size, 64), ~uint64_t{0}) {
  // ids beyond `size` in the last word are never free
  const size_t rem = size % 64;
  if (rem && !free_bits_.empty()) free_bits_.back() = (uint64_t{1} << rem) - 1;
}

uint64_t IdPool::allocate() {
  ScopedLock g(mu_);
  for (size_t w = 0; w < free_bits_.size(); ++w) {
    if (free_bits_[w]) {
      const int bit = __builtin_ffsll(static_cast<long long>(free_bits_[w])) - 1;
      free_bits_[w] &= ~(uint64_t{1} << bit);
      return w * 64 + static_cast<uint64_t>(bit);
    }
  }
  return ID_NONE;
}

void IdPool::free_id(uint64_t id) {
  ScopedLock g(mu_);
  if (id >= size_) throw std::logic_error("IdPool: id out of range");
  const uint64_t m = uint64_t{1} << (id % 64);
  if (free_bits_[id / 64] & m) throw std::logic_error("IdPool: double free");
  free_bits_[id / 64] |= m;
}

size_t IdPool::in_use() const {
  ScopedLock g(mu_);
  size_t free_cnt = 0;
  for (uint64_t w : free_bits_) free_cnt += static_cast<size_t>(__builtin_popcountll(w));
  return size_ - free_cnt;
}

}  // namespace b200net
