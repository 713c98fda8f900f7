// Loads a tuning_data.json through VariantSelector and prints the variant it selects:
//   tuning_rules_check <file> <operator> <backend> <default> <dim>...
#include <cstdlib>
#include <iostream>
#include <memory>
#include <vector>

#include "cut_api.h"

// the operator API links against a backend factory; this tool never creates a Runtime
namespace cut {
std::unique_ptr<ComputeInterface> createB200Compute(int) { return nullptr; }
}  // namespace cut

int main(int argc, char **argv) {
  if (argc < 6) return 2;
  auto &vs = cut::VariantSelector::instance();
  if (!vs.loadFromFile(argv[1])) {
    std::cout << "load failed" << std::endl;
    return 1;
  }
  std::vector<uint32_t> shape;
  for (int i = 5; i < argc; ++i) shape.push_back((uint32_t)std::strtoul(argv[i], nullptr, 10));
  std::cout << vs.select(argv[2], shape, std::atoi(argv[4]), argv[3]) << std::endl;
  return 0;
}
