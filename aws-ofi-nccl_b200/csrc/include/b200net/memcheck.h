// Memory-state annotations for pooled memory. Under AddressSanitizer the calls poison/unpoison
// the ranges so use-after-free of a freelist entry and overruns into its redzone are caught;
// otherwise they compile to nothing (reference: include/nccl_ofi_memcheck*.h).
#pragma once
#include <cstddef>

#if defined(__SANITIZE_ADDRESS__)
#define B200NET_ASAN 1
#elif defined(__has_feature)
#if __has_feature(address_sanitizer)
#define B200NET_ASAN 1
#endif
#endif

#ifdef B200NET_ASAN
extern "C" void __asan_poison_memory_region(void const volatile*, size_t);
extern "C" void __asan_unpoison_memory_region(void const volatile*, size_t);
#endif

namespace b200net::memcheck {
constexpr size_t GRANULARITY = 8;  // poisoning works on 8-byte units
#ifdef B200NET_ASAN
constexpr size_t REDZONE = 16;
inline void make_noaccess(void* p, size_t n) { __asan_poison_memory_region(p, n); }
inline void make_undefined(void* p, size_t n) { __asan_unpoison_memory_region(p, n); }
inline void make_defined(void* p, size_t n) { __asan_unpoison_memory_region(p, n); }
#else
constexpr size_t REDZONE = 0;
inline void make_noaccess(void*, size_t) {}
inline void make_undefined(void*, size_t) {}
inline void make_defined(void*, size_t) {}
#endif
}  // namespace b200net::memcheck
