// Clang thread-safety-analysis annotations; expand to nothing on other compilers
// (reference: include/nccl_ofi_tsa.h).
#pragma once
#if defined(__clang__) && defined(B200NET_THREAD_ANALYSIS)
#define B200NET_TSA(x) __attribute__((x))
#else
#define B200NET_TSA(x)
#endif
#define TSA_CAPABILITY(x) B200NET_TSA(capability(x))
#define TSA_SCOPED_CAPABILITY B200NET_TSA(scoped_lockable)
#define TSA_GUARDED_BY(x) B200NET_TSA(guarded_by(x))
#define TSA_PT_GUARDED_BY(x) B200NET_TSA(pt_guarded_by(x))
#define TSA_ACQUIRE(...) B200NET_TSA(acquire_capability(__VA_ARGS__))
#define TSA_RELEASE(...) B200NET_TSA(release_capability(__VA_ARGS__))
#define TSA_TRY_ACQUIRE(...) B200NET_TSA(try_acquire_capability(__VA_ARGS__))
#define TSA_REQUIRES(...) B200NET_TSA(requires_capability(__VA_ARGS__))
#define TSA_EXCLUDES(...) B200NET_TSA(locks_excluded(__VA_ARGS__))
#define TSA_NO_ANALYSIS B200NET_TSA(no_thread_safety_analysis)
