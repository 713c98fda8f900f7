// Minimal assertion helpers for the C++ test executables (GoogleTest is not
// available offline).  Each CHECK prints file:line on failure; main() returns
// the number of failed checks.
#pragma once
#include <cmath>
#include <cstdio>
#include <functional>
#include <stdexcept>
#include <string>

static int g_failures = 0;
static int g_checks = 0;

#define CHECK(cond)                                                        \
  do {                                                                     \
    ++g_checks;                                                            \
    if (!(cond)) {                                                         \
      ++g_failures;                                                        \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);          \
    }                                                                      \
  } while (0)

#define CHECK_NEAR(a, b, tol)                                                                  \
  do {                                                                                         \
    ++g_checks;                                                                                \
    const double _a = (a), _b = (b), _t = (tol);                                               \
    if (!(std::fabs(_a - _b) <= _t)) {                                                         \
      ++g_failures;                                                                            \
      std::printf("FAIL %s:%d: |%s - %s| = |%g - %g| > %g\n", __FILE__, __LINE__, #a, #b, _a, _b, _t); \
    }                                                                                          \
  } while (0)

// Expects `fn` to throw std::runtime_error whose message contains `needle`.
inline void checkThrows(const char *file, int line, const std::function<void()> &fn, const std::string &needle) {
  ++g_checks;
  try {
    fn();
  } catch (const std::runtime_error &e) {
    if (std::string(e.what()).find(needle) != std::string::npos) return;
    ++g_failures;
    std::printf("FAIL %s:%d: threw \"%s\", expected it to contain \"%s\"\n", file, line, e.what(), needle.c_str());
    return;
  }
  ++g_failures;
  std::printf("FAIL %s:%d: did not throw (expected \"%s\")\n", file, line, needle.c_str());
}
#define CHECK_THROWS(stmt, needle) checkThrows(__FILE__, __LINE__, [&]() { stmt; }, needle)

#define RUN(fn)                          \
  do {                                   \
    const int before = g_failures;       \
    fn();                                \
    std::printf("%s %s\n", g_failures == before ? "ok  " : "FAIL", #fn); \
  } while (0)

inline int finish() {
  std::printf("%d checks, %d failures\n", g_checks, g_failures);
  return g_failures ? 1 : 0;
}
