// Integer helpers used across the plugin (reference: include/nccl_ofi_math.h).
#pragma once
#include <cstddef>
#include <cstdint>

namespace b200net {

template <typename T>
constexpr T div_ceil(T x, T y) { return (x + y - 1) / y; }
template <typename T>
constexpr bool is_pow2(T x) { return x != 0 && (x & (x - 1)) == 0; }
template <typename T>
constexpr T round_down(T x, T align) { return x - (x % align); }
template <typename T>
constexpr T round_up(T x, T align) { return div_ceil(x, align) * align; }
template <typename T>
constexpr T round_up_pow2_align(T x, T pow2) { return (x + pow2 - 1) & ~(pow2 - 1); }
constexpr bool is_aligned(uintptr_t x, uintptr_t a) { return (x % a) == 0; }
inline bool is_ptr_aligned(const void* p, uintptr_t a) { return is_aligned(reinterpret_cast<uintptr_t>(p), a); }
constexpr uint64_t next_pow2(uint64_t x) {
  if (x <= 1) return 1;
  --x;
  x |= x >> 1; x |= x >> 2; x |= x >> 4; x |= x >> 8; x |= x >> 16; x |= x >> 32;
  return x + 1;
}
constexpr unsigned log2_floor(uint64_t x) {
  unsigned r = 0;
  while (x >>= 1) ++r;
  return r;
}
template <typename T>
constexpr T clamp_to(T v, T lo, T hi) { return v < lo ? lo : (v > hi ? hi : v); }

}  // namespace b200net
