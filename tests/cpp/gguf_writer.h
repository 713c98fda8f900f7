// Minimal GGUF v3 writer for the C++ tests (test infrastructure): header, metadata pairs appended by the
// caller, tensor directory entries, then the data section at the file's alignment.
#pragma once
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

struct GGUFWriter {
  std::vector<uint8_t> b;
  template <typename T> void put(T v) {
    const uint8_t *p = reinterpret_cast<const uint8_t *>(&v);
    b.insert(b.end(), p, p + sizeof(T));
  }
  void str(const std::string &s) {
    put<uint64_t>(s.size());
    b.insert(b.end(), s.begin(), s.end());
  }
  void header(uint64_t tensors, uint64_t metaPairs) {
    put<uint32_t>(0x46554747u);
    put<uint32_t>(3);
    put<uint64_t>(tensors);
    put<uint64_t>(metaPairs);
  }
  void tensor2d(const std::string &name, uint64_t cols, uint64_t rows, uint32_t type, uint64_t offset) {
    str(name);
    put<uint32_t>(2);
    put<uint64_t>(cols);
    put<uint64_t>(rows);
    put<uint32_t>(type);
    put<uint64_t>(offset);
  }
  bool save(const std::string &path) const {
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const bool ok = fwrite(b.data(), 1, b.size(), f) == b.size();
    fclose(f);
    return ok;
  }
};
