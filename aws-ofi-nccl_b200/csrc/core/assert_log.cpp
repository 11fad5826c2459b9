// assert_always + logger plumbing.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <string>

#include "b200net/assert.h"
#include "b200net/log.h"

namespace b200net {

void assert_fail(const char* expr, const char* file, int line) {
  std::string msg = std::string("assertion failed: ") + expr + " at " + file + ":" + std::to_string(line);
  NET_WARN("%s", msg.c_str());
  throw std::logic_error(msg);
}

ncclDebugLogger_t g_log_fn = nullptr;
static std::atomic<int> g_warns{0};

void set_logger(ncclDebugLogger_t fn) { g_log_fn = fn; }
int log_warn_count() { return g_warns.load(); }
void log_note_warn() { g_warns.fetch_add(1); }

void stderr_logger(ncclDebugLogLevel level, unsigned long, const char* file, int line, const char* fmt, ...) {
  static const int verbosity = [] {
    const char* e = getenv("B200NET_LOG_LEVEL");
    if (!e) e = getenv("NCCL_DEBUG");
    if (!e) return 2;
    std::string s(e);
    if (s == "TRACE" || s == "5") return 5;
    if (s == "INFO" || s == "3") return 3;
    if (s == "WARN" || s == "2") return 2;
    if (s == "NONE" || s == "0") return 0;
    return 2;
  }();
  if (static_cast<int>(level) > verbosity && level != NCCL_LOG_ABORT) return;
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  const char* tag = level == NCCL_LOG_WARN ? "WARN" : level == NCCL_LOG_INFO ? "INFO" : level == NCCL_LOG_TRACE ? "TRACE" : "LOG";
  fprintf(stderr, "[%s] %s (%s:%d)\n", tag, buf, file, line);
}

}  // namespace b200net
