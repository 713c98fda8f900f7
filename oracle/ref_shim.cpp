// ref_shim.cpp -- thin C entry points over the reference's own GGUF reader.
//
// TEST INFRASTRUCTURE ONLY.  Compiled together with the reference's unmodified
// interface/loader/gguf/gguf_reader.cpp (found through REF_ROOT at build time,
// never copied into this repository) into oracle/_ref/libcutref.so.  It lets
// the tests and the fixture generator run the reference's CPU dequantisers
// (GGUFReader::read_tensor_f32 -> dequantize_q8_0 / q4_0 / q4_k, which are
// private statics) and its plane separation (read_tensor_q8_separated /
// read_tensor_q4_separated) on a GGUF file.  Returns 0 on success, a negative
// code on failure with the message retrievable through cutref_last_error().
#include "gguf_reader.hpp"

#include <cstring>
#include <string>

static thread_local std::string g_err;

extern "C" {

__attribute__((visibility("default"))) const char *cutref_last_error() { return g_err.c_str(); }

__attribute__((visibility("default"))) long cutref_tensor_elements(const char *path, const char *name) {
  try {
    gguf::GGUFReader r(path);
    return static_cast<long>(r.get_tensor_info(name).n_elements());
  } catch (const std::exception &e) {
    g_err = e.what();
    return -1;
  }
}

// Dequantise tensor `name` of the file at `path` into out[capacity] floats.
__attribute__((visibility("default"))) int cutref_read_f32(const char *path, const char *name, float *out, size_t capacity) {
  try {
    gguf::GGUFReader r(path);
    std::vector<float> v = r.read_tensor_f32(name);
    if (v.size() > capacity) {
      g_err = "output buffer too small";
      return -2;
    }
    std::memcpy(out, v.data(), v.size() * sizeof(float));
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return -1;
  }
}

__attribute__((visibility("default"))) int cutref_read_q8_separated(const char *path, const char *name, int8_t *values, uint16_t *scales,
                             uint32_t *rows, uint32_t *cols) {
  try {
    gguf::GGUFReader r(path);
    auto s = r.read_tensor_q8_separated(name);
    std::memcpy(values, s.values.data(), s.values.size());
    std::memcpy(scales, s.scales.data(), s.scales.size() * sizeof(uint16_t));
    *rows = s.rows;
    *cols = s.cols;
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return -1;
  }
}

__attribute__((visibility("default"))) int cutref_read_q4_separated(const char *path, const char *name, uint8_t *packed, uint16_t *scales,
                             uint32_t *rows, uint32_t *cols) {
  try {
    gguf::GGUFReader r(path);
    auto s = r.read_tensor_q4_separated(name);
    std::memcpy(packed, s.packedValues.data(), s.packedValues.size());
    std::memcpy(scales, s.scales.data(), s.scales.size() * sizeof(uint16_t));
    *rows = s.rows;
    *cols = s.cols;
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return -1;
  }
}

}  // extern "C"
