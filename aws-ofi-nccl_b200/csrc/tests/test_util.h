// Minimal harness for the C++ unit tests: each test is a program, exit status 0 = pass.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <stdexcept>

static int g_failures = 0;
#define CHECK(cond)                                                              \
  do {                                                                           \
    if (!(cond)) {                                                               \
      fprintf(stderr, "%s:%d CHECK failed: %s\n", __FILE__, __LINE__, #cond);    \
      ++g_failures;                                                              \
    }                                                                            \
  } while (0)
#define CHECK_EQ(a, b)                                                                              \
  do {                                                                                              \
    auto _a = (a);                                                                                  \
    auto _b = (b);                                                                                  \
    if (!(_a == _b)) {                                                                              \
      fprintf(stderr, "%s:%d CHECK_EQ failed: %s (%lld) vs %s (%lld)\n", __FILE__, __LINE__, #a,    \
              (long long)_a, #b, (long long)_b);                                                    \
      ++g_failures;                                                                                 \
    }                                                                                               \
  } while (0)
#define CHECK_THROWS(stmt)                                                              \
  do {                                                                                  \
    bool _thrown = false;                                                               \
    try { stmt; } catch (const std::exception&) { _thrown = true; }                     \
    if (!_thrown) {                                                                     \
      fprintf(stderr, "%s:%d expected an exception: %s\n", __FILE__, __LINE__, #stmt);  \
      ++g_failures;                                                                     \
    }                                                                                   \
  } while (0)
#define TEST_MAIN_END()                                           \
  do {                                                            \
    if (g_failures) {                                             \
      fprintf(stderr, "%d check(s) failed\n", g_failures);        \
      return 1;                                                   \
    }                                                             \
    printf("ok\n");                                               \
    return 0;                                                     \
  } while (0)
