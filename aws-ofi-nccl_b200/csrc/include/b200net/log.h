// Logging through NCCL's logger callback with a fixed prefix; falls back to stderr when the
// plugin is driven without NCCL (unit tests, the Python tools). TRACE compiles out unless
// B200NET_ENABLE_TRACE is defined (reference: include/nccl_ofi_log.h).
#pragma once
#include "nccl_abi.h"

namespace b200net {
extern ncclDebugLogger_t g_log_fn;  // installed by init(); may be null
void set_logger(ncclDebugLogger_t fn);
void stderr_logger(ncclDebugLogLevel level, unsigned long flags, const char* file, int line, const char* fmt, ...);
int log_warn_count();  // number of WARN lines emitted so far (tests use it)
void log_note_warn();
}  // namespace b200net

#define B200NET_LOG(level, flags, fmt, ...)                                                              \
  do {                                                                                                   \
    ::ncclDebugLogger_t _fn = ::b200net::g_log_fn ? ::b200net::g_log_fn : ::b200net::stderr_logger;     \
    _fn(level, flags, __FILE__, __LINE__, "NET/B200 " fmt, ##__VA_ARGS__);                               \
  } while (0)
#define NET_WARN(fmt, ...) \
  do { ::b200net::log_note_warn(); B200NET_LOG(NCCL_LOG_WARN, NCCL_ALL, fmt, ##__VA_ARGS__); } while (0)
#define NET_INFO(flags, fmt, ...) B200NET_LOG(NCCL_LOG_INFO, flags, fmt, ##__VA_ARGS__)
#ifdef B200NET_ENABLE_TRACE
#define NET_TRACE(flags, fmt, ...) B200NET_LOG(NCCL_LOG_TRACE, flags, fmt, ##__VA_ARGS__)
#else
#define NET_TRACE(flags, fmt, ...) do { } while (0)
#endif
