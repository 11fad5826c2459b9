// assert_always: an assertion that survives NDEBUG and throws instead of aborting, so the
// validated API layer can turn it into an ncclResult_t (reference: include/nccl_ofi_assert.h).
#pragma once
#include <stdexcept>
#include <string>

namespace b200net {
[[noreturn]] void assert_fail(const char* expr, const char* file, int line);
}
#define B200NET_ASSERT_ALWAYS(expr) \
  do { if (!(expr)) ::b200net::assert_fail(#expr, __FILE__, __LINE__); } while (0)
