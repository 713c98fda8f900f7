// ref_runner_shim.cpp -- C entry points over the file-static re-encoders of the reference's runner.
//
// TEST INFRASTRUCTURE ONLY.  The reference's interface/runner/llama/llama.cpp keeps its weight
// re-encoders (f32ToF16, f16ToF32, quantizeRowsQ8_0, requantizeQ4KToAffine) file-static, so they
// can only be reached from inside that translation unit: this file #includes it, unmodified, from
// where it lies under REF_ROOT at build time (never copied into this repository) and exports thin
// wrappers.  Everything else of the unit is discarded at link time (--gc-sections), so the library
// needs none of the reference's runtime.  Built into oracle/_ref/libcutref_runner.so; used to pin
// the C restatements of oracle/cut_oracle.c bit for bit.
#include "llama.cpp"

#define SHIM_API extern "C" __attribute__((visibility("default"), used))

SHIM_API uint16_t cutref_runner_f32_to_f16(float v) { return gguf::f32ToF16(v); }
SHIM_API float cutref_runner_f16_to_f32(uint16_t h) { return gguf::f16ToF32(h); }

// n floats (a multiple of 32) -> n int8 values + n / 32 fp16 scales
SHIM_API void cutref_runner_quantize_rows_q8_0(const float *x, size_t n, int8_t *values, uint16_t *scales) {
  std::vector<float> in(x, x + n);
  std::vector<int8_t> v;
  std::vector<uint16_t> s;
  gguf::quantizeRowsQ8_0(in, v, s);
  std::memcpy(values, v.data(), v.size());
  std::memcpy(scales, s.data(), s.size() * sizeof(uint16_t));
}

// raw Q4_K tensor [N rows, K] -> packedT [K, N / 2] and scalesT [2 K / 32, N]; 1 on success, 0 when the
// reference declines the shape.  packed_cap / scales_cap: capacities in elements.
SHIM_API int cutref_runner_requant_q4k_affine(const uint8_t *raw, size_t raw_bytes, uint32_t N, uint32_t K, uint8_t *packedT,
                                              size_t packed_cap, uint16_t *scalesT, size_t scales_cap, size_t *packed_size,
                                              size_t *scales_size) {
  std::vector<uint8_t> in(raw, raw + raw_bytes), p;
  std::vector<uint16_t> s;
  if (!gguf::requantizeQ4KToAffine(in, N, K, p, s)) return 0;
  *packed_size = p.size();
  *scales_size = s.size();
  if (p.size() > packed_cap || s.size() > scales_cap) return -1;
  std::memcpy(packedT, p.data(), p.size());
  std::memcpy(scalesT, s.data(), s.size() * sizeof(uint16_t));
  return 1;
}
