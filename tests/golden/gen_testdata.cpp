// Emits the pseudo-random activation vectors the reference's tests draw, so the
// replayed known-answer cases use bit-identical inputs.  Restates
// generateTestData<float> (tests/harness/OpRefs.h:241-266: std::mt19937(seed),
// uniform_real_distribution<float>(0.1, 10)) and the generator of the
// model-geometry tests (tests/runtime/RuntimeTests.cpp:2865-2868:
// std::mt19937(42), uniform_real_distribution<float>(-1, 1)).
// Usage: gen_testdata <lo> <hi> <seed> <count>  -> raw float32 on stdout.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

int main(int argc, char **argv) {
  if (argc != 5) return 2;
  float lo = std::strtof(argv[1], nullptr), hi = std::strtof(argv[2], nullptr);
  unsigned seed = static_cast<unsigned>(std::strtoul(argv[3], nullptr, 10));
  size_t count = std::strtoull(argv[4], nullptr, 10);
  std::mt19937 gen(seed);
  std::uniform_real_distribution<float> dist(lo, hi);
  std::vector<float> v(count);
  for (auto &x : v) x = dist(gen);
  std::fwrite(v.data(), sizeof(float), v.size(), stdout);
  return 0;
}
