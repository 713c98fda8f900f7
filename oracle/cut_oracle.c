/*
 * cut_oracle.c -- CPU restatement of the reference's GGUF quantized-matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against; nothing in the product library links, loads or calls it.  Only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg use it.
 *
 * Every function restates one piece of the reference (trviv/cut) and names the
 * reference file:line it follows.  Parity of this restatement is pinned three
 * ways: against the reference's own in-code known-answer tests
 * (tests/harness/OpRegistry.h, tests/runtime/*.cpp), against the
 * reference's gguf_reader.cpp compiled unmodified (oracle/Makefile ->
 * oracle/_ref/libcutref.so), and -- for the runner's weight re-encoders, which
 * the reference keeps file-static and does not test -- against those very
 * functions, reached by compiling its runner translation unit
 * (oracle/ref_runner_shim.cpp -> oracle/_ref/libcutref_runner.so).
 *
 * Plain C99, no dependencies beyond libm.  Optional OpenMP (-fopenmp) only
 * parallelises the outer row loops of the matmul helpers; results do not
 * depend on the thread count.  Build with -ffp-contract=off: the reference's
 * CPU code is compiled without fused multiply-add, and bit-exactness of the
 * dequantised values is defined against that.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* fp16 <-> fp32                                                             */
/* ------------------------------------------------------------------------- */

/* interface/loader/gguf/gguf_reader.cpp:515-539 -- half bits to float,
 * subnormals decoded as mantissa * 2^-24, inf/NaN passed through. */
ORC_API float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exponent = ((uint32_t)h & 0x7C00u) >> 10;
  uint32_t mantissa = ((uint32_t)h & 0x03FFu) << 13;
  float out;
  if (exponent == 0) {
    if (mantissa == 0) {
      memcpy(&out, &sign, sizeof(out));
      return out;
    }
    out = (float)(h & 0x03FFu) * 5.960464477539063e-08f;
    return (h & 0x8000u) ? -out : out;
  }
  if (exponent == 31) {
    if (mantissa) return NAN;
    return (h & 0x8000u) ? -INFINITY : INFINITY;
  }
  uint32_t bits = sign | ((exponent + 112u) << 23) | mantissa;
  memcpy(&out, &bits, sizeof(out));
  return out;
}

/* interface/runner/llama/llama.cpp:445-482 -- the runner's float -> half:
 * round half UP on the dropped bits (not ties-to-even), subnormals encoded,
 * overflow clamps to infinity. */
ORC_API uint16_t orc_f32_to_f16_runner(float v) {
  uint32_t u;
  memcpy(&u, &v, sizeof(u));
  uint32_t sign = (u >> 16) & 0x8000u;
  int32_t e = (int32_t)((u >> 23) & 0xffu) - 127 + 15;
  uint32_t mantissa = u & 0x7fffffu;
  if (e <= 0) {
    uint32_t shift = (uint32_t)(14 - e);
    if (shift > 24) return (uint16_t)sign;
    uint32_t significand = 0x800000u | mantissa;
    uint32_t half = significand >> shift;
    if ((significand >> (shift - 1)) & 1u) ++half;
    return (uint16_t)(sign | half);
  }
  if (e >= 31) return (uint16_t)(sign | 0x7c00u);
  uint32_t m = mantissa >> 13;
  if (mantissa & 0x1000u) {
    ++m;
    if (m == 0x400u) {
      m = 0;
      ++e;
      if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    }
  }
  return (uint16_t)(sign | ((uint32_t)e << 10) | m);
}

/* tests/harness/OpRefs.h:164-177 -- the test helper's float -> half:
 * truncates the mantissa and flushes subnormals to zero. */
ORC_API uint16_t orc_f32_to_f16_trunc(float value) {
  uint32_t f32;
  memcpy(&f32, &value, sizeof(f32));
  uint32_t sign = (f32 >> 16) & 0x8000u;
  int32_t exponent = (int32_t)((f32 >> 23) & 0xFFu) - 127 + 15;
  uint32_t mantissa = (f32 >> 13) & 0x03FFu;
  if (exponent <= 0) return (uint16_t)sign;
  if (exponent >= 31) return (uint16_t)(sign | 0x7C00u);
  return (uint16_t)(sign | ((uint32_t)exponent << 10) | mantissa);
}

ORC_API void orc_f16_to_f32_array(const uint16_t *in, float *out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = orc_f16_to_f32(in[i]);
}

/* ------------------------------------------------------------------------- */
/* GGUF block dequantisation (native block layout)                           */
/* ------------------------------------------------------------------------- */

/* interface/loader/gguf/gguf_reader.cpp:826-850 -- Q8_0: 34-byte blocks of
 * {f16 d, int8 q[32]}, value = float(q) * d. */
ORC_API void orc_dequant_q8_0(const uint8_t *data, float *out, size_t n_elements) {
  size_t n_blocks = (n_elements + 31) / 32;
  size_t o = 0;
  for (size_t i = 0; i < n_blocks && o < n_elements; ++i) {
    const uint8_t *blk = data + i * 34;
    uint16_t dbits;
    memcpy(&dbits, blk, 2);
    float d = orc_f16_to_f32(dbits);
    for (size_t j = 0; j < 32 && o < n_elements; ++j) {
      out[o++] = (float)(int8_t)blk[2 + j] * d;
    }
  }
}

/* interface/loader/gguf/gguf_reader.cpp:541-572 -- Q4_0: 18-byte blocks of
 * {f16 d, 16 bytes}; byte j holds element j (low nibble) and element j+16
 * (high nibble); value = float(nibble - 8) * d. */
ORC_API void orc_dequant_q4_0(const uint8_t *data, float *out, size_t n_elements) {
  size_t n_blocks = (n_elements + 31) / 32;
  for (size_t i = 0; i < n_blocks; ++i) {
    const uint8_t *blk = data + i * 18;
    uint16_t dbits;
    memcpy(&dbits, blk, 2);
    float d = orc_f16_to_f32(dbits);
    size_t base = i * 32;
    for (size_t j = 0; j < 16; ++j) {
      uint8_t byte = blk[2 + j];
      int x0 = (int)(byte & 0x0F) - 8;
      int x1 = (int)((byte >> 4) & 0x0F) - 8;
      if (base + j < n_elements) out[base + j] = (float)x0 * d;
      if (base + j + 16 < n_elements) out[base + j + 16] = (float)x1 * d;
    }
  }
}

/* interface/loader/gguf/gguf_reader.cpp:668-676 -- 6-bit scale/min of
 * sub-block j from the 12 packed bytes of a Q4_K super-block. */
static void orc_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
  if (j < 4) {
    *sc = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

ORC_API void orc_get_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
  orc_scale_min_k4(j, q, sc, m);
}

/* interface/loader/gguf/gguf_reader.cpp:678-724 -- Q4_K: 144-byte super-blocks
 * {f16 d, f16 dmin, 12 bytes scales, 128 bytes qs}; four 64-element groups,
 * low nibbles first then high nibbles; value = (d*sc)*q - (dmin*m) with the
 * two products formed in float before the subtract. */
ORC_API void orc_dequant_q4_k(const uint8_t *data, float *out, size_t n_elements) {
  size_t n_blocks = (n_elements + 255) / 256;
  size_t o = 0;
  for (size_t i = 0; i < n_blocks && o < n_elements; ++i) {
    const uint8_t *blk = data + i * 144;
    uint16_t dbits, mbits;
    memcpy(&dbits, blk, 2);
    memcpy(&mbits, blk + 2, 2);
    float d = orc_f16_to_f32(dbits);
    float dmin = orc_f16_to_f32(mbits);
    const uint8_t *scales = blk + 4;
    const uint8_t *qs = blk + 16;
    int is = 0;
    for (int j = 0; j < 256 && o < n_elements; j += 64) {
      uint8_t sc1, m1, sc2, m2;
      orc_scale_min_k4(is, scales, &sc1, &m1);
      float d1 = d * (float)sc1;
      float dm1 = dmin * (float)m1;
      orc_scale_min_k4(is + 1, scales, &sc2, &m2);
      float d2 = d * (float)sc2;
      float dm2 = dmin * (float)m2;
      for (int l = 0; l < 32 && o < n_elements; ++l) {
        float p = d1 * (float)(qs[l] & 0xF);
        out[o++] = p - dm1;
      }
      for (int l = 0; l < 32 && o < n_elements; ++l) {
        float p = d2 * (float)((qs[l] >> 4) & 0xF);
        out[o++] = p - dm2;
      }
      qs += 32;
      is += 2;
    }
  }
}

/* interface/loader/gguf/gguf_reader.cpp:726-772 -- Q5_K: 176-byte super-blocks
 * {f16 d, f16 dmin, 12 bytes scales, 32 bytes qh, 128 bytes ql}; four groups of
 * 64 elements, low nibbles then high nibbles of the group's 32 ql bytes; bit
 * 2g (2g+1) of qh[l] is the fifth bit of element l of the low (high) half;
 * value = (d*sc)*q - (dmin*m), the products formed in float before the subtract. */
ORC_API void orc_dequant_q5_k(const uint8_t *data, float *out, size_t n_elements) {
  size_t n_blocks = (n_elements + 255) / 256;
  size_t o = 0;
  for (size_t i = 0; i < n_blocks && o < n_elements; ++i) {
    const uint8_t *blk = data + i * 176;
    uint16_t dbits, mbits;
    memcpy(&dbits, blk, 2);
    memcpy(&mbits, blk + 2, 2);
    float d = orc_f16_to_f32(dbits);
    float dmin = orc_f16_to_f32(mbits);
    const uint8_t *scales = blk + 4;
    const uint8_t *qh = blk + 16;
    const uint8_t *ql = blk + 48;
    for (int g = 0; g < 4 && o < n_elements; ++g) {
      uint8_t sc1, m1, sc2, m2;
      orc_scale_min_k4(2 * g, scales, &sc1, &m1);
      orc_scale_min_k4(2 * g + 1, scales, &sc2, &m2);
      float d1 = d * (float)sc1, dm1 = dmin * (float)m1;
      float d2 = d * (float)sc2, dm2 = dmin * (float)m2;
      uint8_t u1 = (uint8_t)(1u << (2 * g)), u2 = (uint8_t)(2u << (2 * g));
      for (int l = 0; l < 32 && o < n_elements; ++l) {
        float p = d1 * (float)((ql[32 * g + l] & 0xF) + ((qh[l] & u1) ? 16 : 0));
        out[o++] = p - dm1;
      }
      for (int l = 0; l < 32 && o < n_elements; ++l) {
        float p = d2 * (float)((ql[32 * g + l] >> 4) + ((qh[l] & u2) ? 16 : 0));
        out[o++] = p - dm2;
      }
    }
  }
}

/* interface/loader/gguf/gguf_reader.cpp:774-824 -- Q6_K: 210-byte super-blocks
 * {128 bytes ql, 64 bytes qh, 16 int8 scales, f16 d}; two halves of 128
 * elements, each four interleaved runs of 32: run r of element l takes its low
 * four bits from ql[l + 32 (r & 1)] (low nibble for r < 2, high nibble else) and
 * its two high bits from bits 2r..2r+1 of qh[l]; the 6-bit value is biased by 32;
 * scale index = 8 half + 2 r + l / 16; value = (d * sc) * q.  Whole super-blocks
 * only (the reference's partial-block tail is not restated). */
ORC_API void orc_dequant_q6_k(const uint8_t *data, float *out, size_t n_elements) {
  size_t n_blocks = n_elements / 256;
  for (size_t i = 0; i < n_blocks; ++i) {
    const uint8_t *blk = data + i * 210;
    uint16_t dbits;
    memcpy(&dbits, blk + 208, 2);
    float d = orc_f16_to_f32(dbits);
    for (int half = 0; half < 2; ++half) {
      const uint8_t *ql = blk + 64 * half;
      const uint8_t *qh = blk + 128 + 32 * half;
      const int8_t *sc = (const int8_t *)(blk + 192 + 8 * half);
      float *o = out + i * 256 + 128 * half;
      for (int l = 0; l < 32; ++l) {
        int is = l / 16;
        for (int r = 0; r < 4; ++r) {
          uint8_t lo = ql[l + 32 * (r & 1)];
          int q = (int)((r < 2 ? (lo & 0xF) : (lo >> 4)) | (((qh[l] >> (2 * r)) & 3) << 4)) - 32;
          float ds = d * (float)sc[is + 2 * r];
          o[l + 32 * r] = ds * (float)q;
        }
      }
    }
  }
}

/* interface/loader/gguf/gguf_reader.cpp:860-870 -- BF16: the upper 16 bits of a float32. */
ORC_API void orc_dequant_bf16(const uint8_t *data, float *out, size_t n_elements) {
  for (size_t i = 0; i < n_elements; ++i) {
    uint16_t b;
    memcpy(&b, data + 2 * i, 2);
    uint32_t w = (uint32_t)b << 16;
    memcpy(out + i, &w, 4);
  }
}

/* Format codes shared with the tests (they mirror the product's C ABI values
 * but are defined independently here).  Q5_K, Q6_K and BF16 exist for the
 * dequant operator only. */
/* interface/loader/gguf/gguf_reader.cpp:574-611 -- Q4_1: 20-byte blocks of {f16 d, f16 m, 16 bytes};
 * byte j holds element j (low nibble) and element j + 16 (high nibble); value = float(nibble) * d + m
 * (the product and the sum each rounded: the reference's CPU build does not contract). */
ORC_API void orc_dequant_q4_1(const uint8_t *data, float *out, size_t n_elements) {
  size_t n_blocks = (n_elements + 31) / 32;
  for (size_t i = 0; i < n_blocks; ++i) {
    const uint8_t *blk = data + i * 20;
    uint16_t dbits, mbits;
    memcpy(&dbits, blk, 2);
    memcpy(&mbits, blk + 2, 2);
    float d = orc_f16_to_f32(dbits), m = orc_f16_to_f32(mbits);
    size_t base = i * 32;
    for (size_t j = 0; j < 16; ++j) {
      uint8_t byte = blk[4 + j];
      int x0 = byte & 0x0F, x1 = (byte >> 4) & 0x0F;
      if (base + j < n_elements) out[base + j] = (float)x0 * d + m;
      if (base + j + 16 < n_elements) out[base + j + 16] = (float)x1 * d + m;
    }
  }
}

/* interface/loader/gguf/gguf_reader.cpp:613-660 -- Q5_0: 22-byte blocks of {f16 d, u32 qh, 16 bytes};
 * nibbles as in Q4_0, bit j of qh is the fifth bit of element j, bit j + 16 that of element j + 16;
 * value = float(q5 - 16) * d. */
ORC_API void orc_dequant_q5_0(const uint8_t *data, float *out, size_t n_elements) {
  size_t n_blocks = (n_elements + 31) / 32;
  for (size_t i = 0; i < n_blocks; ++i) {
    const uint8_t *blk = data + i * 22;
    uint16_t dbits;
    uint32_t qh;
    memcpy(&dbits, blk, 2);
    memcpy(&qh, blk + 2, 4);
    float d = orc_f16_to_f32(dbits);
    size_t base = i * 32;
    for (size_t j = 0; j < 16; ++j) {
      uint8_t byte = blk[6 + j];
      int lo = (byte & 0x0F) | (int)(((qh >> j) & 1u) << 4);
      int hi = ((byte >> 4) & 0x0F) | (int)(((qh >> (j + 16)) & 1u) << 4);
      if (base + j < n_elements) out[base + j] = (float)(lo - 16) * d;
      if (base + j + 16 < n_elements) out[base + j + 16] = (float)(hi - 16) * d;
    }
  }
}

enum { ORC_Q8_0 = 0, ORC_Q4_0 = 1, ORC_Q4_K = 2, ORC_Q5_K = 3, ORC_Q6_K = 4, ORC_BF16 = 5, ORC_Q4_1 = 6, ORC_Q5_0 = 7 };

ORC_API size_t orc_block_bytes(int fmt) {
  switch (fmt) {
    case ORC_Q8_0: return 34;
    case ORC_Q4_0: return 18;
    case ORC_Q4_K: return 144;
    case ORC_Q5_K: return 176;
    case ORC_Q6_K: return 210;
    case ORC_Q4_1: return 20;
    case ORC_Q5_0: return 22;
    default: return 2;
  }
}
ORC_API size_t orc_block_elems(int fmt) {
  return (fmt == ORC_Q4_K || fmt == ORC_Q5_K || fmt == ORC_Q6_K) ? 256 : (fmt == ORC_BF16 ? 1 : 32);
}

ORC_API size_t orc_row_bytes(int fmt, size_t K) {
  size_t be = orc_block_elems(fmt);
  return (K + be - 1) / be * orc_block_bytes(fmt);
}

ORC_API void orc_dequant(int fmt, const uint8_t *data, float *out, size_t n_elements) {
  if (fmt == ORC_Q8_0)
    orc_dequant_q8_0(data, out, n_elements);
  else if (fmt == ORC_Q4_0)
    orc_dequant_q4_0(data, out, n_elements);
  else if (fmt == ORC_Q5_K)
    orc_dequant_q5_k(data, out, n_elements);
  else if (fmt == ORC_Q6_K)
    orc_dequant_q6_k(data, out, n_elements);
  else if (fmt == ORC_BF16)
    orc_dequant_bf16(data, out, n_elements);
  else if (fmt == ORC_Q4_1)
    orc_dequant_q4_1(data, out, n_elements);
  else if (fmt == ORC_Q5_0)
    orc_dequant_q5_0(data, out, n_elements);
  else
    orc_dequant_q4_k(data, out, n_elements);
}

/* Row-wise dequant into a [rows, ldo] float matrix (ldo >= cols), the shape
 * the reference's DequantOpNode produces (operators/impl/dequant/DequantOp.cpp:15-17:
 * output stride = cols rounded up to 4; DequantQ4K.cu:12-49). */
ORC_API void orc_dequant_rows(int fmt, const uint8_t *data, float *out, size_t rows, size_t cols,
                              size_t ldo) {
  size_t rb = orc_row_bytes(fmt, cols);
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; ++r) orc_dequant(fmt, data + (size_t)r * rb, out + (size_t)r * ldo, cols);
}

/* ------------------------------------------------------------------------- */
/* Loader-side plane separation and runner-side re-encodes                   */
/* ------------------------------------------------------------------------- */

/* interface/loader/gguf/gguf_reader.cpp:389-444 -- Q8_0 [rows, cols] blocks ->
 * int8 values [rows, cols] + raw f16 scale bits [rows, cols/32]. */
ORC_API void orc_q8_separate(const uint8_t *raw, size_t rows, size_t cols, int8_t *values,
                             uint16_t *scales) {
  size_t bpr = cols / 32, total = rows * bpr;
  for (size_t b = 0; b < total; ++b) {
    const uint8_t *p = raw + b * 34;
    memcpy(&scales[b], p, 2);
    size_t row = b / bpr, bir = b % bpr;
    memcpy(values + row * cols + bir * 32, p + 2, 32);
  }
}

/* interface/loader/gguf/gguf_reader.cpp:446-501 -- Q4_0 [rows, cols] blocks ->
 * packed nibbles [rows, cols/2] (GGML order kept) + f16 scale bits. */
ORC_API void orc_q4_separate(const uint8_t *raw, size_t rows, size_t cols, uint8_t *packed,
                             uint16_t *scales) {
  size_t bpr = cols / 32, total = rows * bpr;
  for (size_t b = 0; b < total; ++b) {
    const uint8_t *p = raw + b * 18;
    memcpy(&scales[b], p, 2);
    size_t row = b / bpr, bir = b % bpr;
    memcpy(packed + row * (cols / 2) + bir * 16, p + 2, 16);
  }
}

/* operators/impl/q4transpose/TransposeQ4Nibble.cu:16-61 with the strides of
 * TransposeQ4NibbleOp.cpp:22-23 -- GGML-packed [N, K/2] (row stride
 * stride_in bytes) -> [K, N/2] (row stride stride_out bytes), low nibble =
 * even n.  Padding bytes of the output rows are left untouched. */
static unsigned orc_read_nibble(const uint8_t *in, size_t stride_in, size_t row, size_t col) {
  size_t blk = col / 32, e = col % 32;
  size_t j = e < 16 ? e : e - 16;
  unsigned hi = e < 16 ? 0u : 1u;
  uint8_t byte = in[row * stride_in + blk * 16 + j];
  return (byte >> (hi * 4u)) & 0xFu;
}

ORC_API void orc_transpose_q4(const uint8_t *in, uint8_t *out, size_t N, size_t K, size_t stride_in,
                              size_t stride_out) {
  size_t halfN = N / 2;
  for (size_t k = 0; k < K; ++k)
    for (size_t bn = 0; bn < halfN; ++bn) {
      size_t n = bn * 2;
      unsigned lo = orc_read_nibble(in, stride_in, n, k);
      unsigned hi = (n + 1 < N) ? orc_read_nibble(in, stride_in, n + 1, k) : 0u;
      out[k * stride_out + bn] = (uint8_t)(lo | (hi << 4));
    }
}

/* Plain 2-D transposes the runner applies to the separated planes
 * (interface/runner/llama/llama.cpp:942-969, 1000-1021): [R, C] -> [C, R]
 * with an output row stride in elements. */
ORC_API void orc_transpose_u16(const uint16_t *in, uint16_t *out, size_t R, size_t C, size_t ldo) {
  for (size_t r = 0; r < R; ++r)
    for (size_t c = 0; c < C; ++c) out[c * ldo + r] = in[r * C + c];
}
ORC_API void orc_transpose_i8(const int8_t *in, int8_t *out, size_t R, size_t C, size_t ldo) {
  for (size_t r = 0; r < R; ++r)
    for (size_t c = 0; c < C; ++c) out[c * ldo + r] = in[r * C + c];
}

/* interface/runner/llama/llama.cpp:573-619 -- Q4_K -> affine 4-bit planes in
 * the matmul's [K, N] orientation: nibbles [K, N/2] (low = even n), scales
 * [2*K/32, N] with rows [0, K/32) = f16(d*sc) and rows [K/32, 2K/32) =
 * f16(8*scale - dmin*m).  Lossy in the two f16 roundings.  Returns 0 when the
 * shape is not re-encodable (K % 256 or N % 2), as the reference does. */
ORC_API int orc_requant_q4k_affine(const uint8_t *raw, size_t raw_bytes, uint32_t N, uint32_t K,
                                   uint8_t *packedT, uint16_t *scalesT) {
  if (K % 256 != 0 || N % 2 != 0) return 0;
  uint32_t blocksK = K / 32;
  size_t superPerRow = K / 256;
  if (raw_bytes < (size_t)N * superPerRow * 144) return 0;
  memset(packedT, 0, (size_t)K * (N / 2));
  memset(scalesT, 0, (size_t)2 * blocksK * N * sizeof(uint16_t));
  for (uint32_t n = 0; n < N; ++n)
    for (uint32_t s = 0; s < superPerRow; ++s) {
      const uint8_t *blk = raw + ((size_t)n * superPerRow + s) * 144;
      uint16_t d, dmin;
      memcpy(&d, blk, 2);
      memcpy(&dmin, blk + 2, 2);
      float fd = orc_f16_to_f32(d), fdmin = orc_f16_to_f32(dmin);
      const uint8_t *scales = blk + 4, *qs = blk + 16;
      for (int g = 0; g < 4; ++g)
        for (int h = 0; h < 2; ++h) {
          uint8_t sc, mm;
          orc_scale_min_k4(2 * g + h, scales, &sc, &mm);
          float scale = fd * (float)sc;
          float t8 = 8.0f * scale;
          float dm = fdmin * (float)mm;
          float minv = t8 - dm;
          uint32_t e0 = s * 256 + (uint32_t)g * 64 + (uint32_t)h * 32;
          uint32_t b = e0 / 32;
          scalesT[(size_t)b * N + n] = orc_f32_to_f16_runner(scale);
          scalesT[((size_t)blocksK + b) * N + n] = orc_f32_to_f16_runner(minv);
          for (uint32_t l = 0; l < 32; ++l) {
            uint8_t byte = qs[g * 32 + l];
            uint8_t q = (h == 0) ? (byte & 0xF) : (uint8_t)(byte >> 4);
            uint32_t k = e0 + l;
            packedT[(size_t)k * (N / 2) + (n >> 1)] |= (uint8_t)(q << ((n & 1) * 4));
          }
        }
    }
  return 1;
}

/* interface/runner/llama/llama.cpp:488-505 -- float rows -> Q8_0 planes:
 * d = amax/127 stored through the runner's f32->f16, q = lround(x / d). */
ORC_API void orc_quantize_rows_q8_0(const float *x, size_t n, int8_t *values, uint16_t *scales) {
  size_t nb = n / 32;
  for (size_t b = 0; b < nb; ++b) {
    const float *p = x + b * 32;
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(p[i]));
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    scales[b] = orc_f32_to_f16_runner(d);
    for (int i = 0; i < 32; ++i) values[b * 32 + i] = (int8_t)lroundf(p[i] * id);
  }
}

/* ------------------------------------------------------------------------- */
/* Fused epilogue                                                            */
/* ------------------------------------------------------------------------- */

/* operators/impl/matmul/MatMulQ4Common.cuh:63-114 -- the unary (type 1) and
 * binary (type 2) epilogues applied to each output element; op codes from
 * operators/runtime/ComputeOpsShared.h:22-66, 118-186. */
ORC_API float orc_epilogue(float v, int fusion_type, int op, float dval) {
  if (fusion_type == 1) {
    float x = v;
    switch (op) {
    case 100: x = -x; break;
    case 101: x = fabsf(x); break;
    case 102: x = sqrtf(x); break;
    case 103: x = x * x; break;
    case 104: x = 1.0f / x; break;
    case 106: x = expf(x); break;
    case 109: x = logf(x); break;
    case 121: x = tanhf(x); break;
    case 122: x = floorf(x); break;
    case 123: x = ceilf(x); break;
    case 124: x = roundf(x); break;
    case 130: x = fmaxf(0.0f, x); break;
    case 131: x = 1.0f / (1.0f + expf(-x)); break;
    case 132: x = x * 0.5f * (1.0f + tanhf(sqrtf(2.0f / 3.14159265f) * (x + 0.044715f * x * x * x))); break;
    case 133: x = x / (1.0f + expf(-x)); break;
    case 134: x = logf(1.0f + expf(x)); break;
    case 137: x = fminf(fmaxf(x, 0.0f), 6.0f); break;
    case 141: x = x * tanhf(logf(1.0f + expf(x))); break;
    case 142: x = x * fminf(fmaxf(x / 6.0f + 0.5f, 0.0f), 1.0f); break;
    case 143: x = fminf(fmaxf(x / 6.0f + 0.5f, 0.0f), 1.0f); break;
    case 148: x = 1.0f / sqrtf(x); break;
    default: break;
    }
    return x;
  }
  if (fusion_type == 2) {
    float a = v, b = dval, r;
    switch (op) {
    case 0: r = a + b; break;
    case 1: r = a - b; break;
    case 2: r = a * b; break;
    case 3: r = a / b; break;
    case 4: r = a - b * floorf(a / b); break;
    case 5: r = powf(a, b); break;
    case 6: r = floorf(a / b); break;
    case 13: r = fminf(a, b); break;
    case 14: r = fmaxf(a, b); break;
    default: r = a + b; break;
    }
    return r;
  }
  return v;
}

/* ------------------------------------------------------------------------- */
/* Quantized matmul, reference plane layout ("[K,N] planes")                 */
/* ------------------------------------------------------------------------- */

/* Element of W in the reference's runtime layout.
 * Q8: operators/impl/matmul/MatMulQ8Common.cuh:127-200 (w = int8 * f16 scale).
 * Q4: operators/impl/matmul/MatMulQ4Common.cuh:126-153 (w = (nib-8)*s, plus
 * min from the lower half of the scales plane when affine). */
static inline float orc_plane_w(int q4, int affine, const uint8_t *B, const uint16_t *S, size_t K,
                                size_t ldb, size_t lds, size_t k, size_t n) {
  float s = orc_f16_to_f32(S[(k >> 5) * lds + n]);
  if (!q4) return (float)(int8_t)B[k * ldb + n] * s;
  uint8_t byte = B[k * ldb + (n >> 1)];
  int v = (int)((byte >> ((n & 1) * 4)) & 0xF) - 8;
  float r = (float)v * s;
  if (affine) {
    size_t blocksK = (K + 31) >> 5;
    r += orc_f16_to_f32(S[((k >> 5) + blocksK) * lds + n]);
  }
  return r;
}

/* C[M,N] = A[M,K] * W over the plane layout.  acc64 = 0 follows the float
 * triple loop of tests/harness/OpRegistry.h:2043-2050; acc64 = 1 the double
 * accumulator of tests/runtime/RuntimeTests.cpp:2907-2920.  lda/ldb/lds/ldc/ldd
 * are row strides in elements (bytes for B); the reference pads each to a
 * multiple of 4 (operators/impl/matmul/MatMulOp.cpp:514-541). */
ORC_API void orc_qmatmul_planes(int q4, int affine, const float *A, const uint8_t *B,
                                const uint16_t *S, float *C, const float *D, size_t M, size_t K,
                                size_t N, size_t lda, size_t ldb, size_t lds, size_t ldc, size_t ldd,
                                int fusion_type, int fusion_op, int acc64) {
#pragma omp parallel for schedule(static)
  for (long nn = 0; nn < (long)N; ++nn) {
    size_t n = (size_t)nn;
    for (size_t m = 0; m < M; ++m) {
      float r;
      if (acc64) {
        double sum = 0.0;
        for (size_t k = 0; k < K; ++k)
          sum += (double)A[m * lda + k] * (double)orc_plane_w(q4, affine, B, S, K, ldb, lds, k, n);
        r = (float)sum;
      } else {
        float sum = 0.0f;
        for (size_t k = 0; k < K; ++k) {
          float p = A[m * lda + k] * orc_plane_w(q4, affine, B, S, K, ldb, lds, k, n);
          sum += p;
        }
        r = sum;
      }
      float dv = (fusion_type == 2 && D) ? D[m * ldd + n] : 0.0f;
      C[m * ldc + n] = orc_epilogue(r, fusion_type, fusion_op, dv);
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Quantized matmul, native GGUF block layout                                */
/* ------------------------------------------------------------------------- */

/* C[M,N] = A[M,K] * dequant(W)^T where W is N rows of GGUF blocks along K.
 * The weights are dequantised exactly as the loader does
 * (gguf_reader.cpp:541-572, 678-724, 826-850) and contracted with the scalar
 * loop of the reference tests (float or double accumulator, see above). */
ORC_API void orc_qmatmul_blocks(int fmt, const float *A, const uint8_t *W, float *C, const float *D,
                                size_t M, size_t K, size_t N, size_t lda, size_t ldc, size_t ldd,
                                int fusion_type, int fusion_op, int acc64) {
  size_t rb = orc_row_bytes(fmt, K);
#pragma omp parallel
  {
    float *w = (float *)malloc(sizeof(float) * (K + 256));
#pragma omp for schedule(static)
    for (long nn = 0; nn < (long)N; ++nn) {
      size_t n = (size_t)nn;
      orc_dequant(fmt, W + n * rb, w, K);
      for (size_t m = 0; m < M; ++m) {
        float r;
        if (acc64) {
          double sum = 0.0;
          for (size_t k = 0; k < K; ++k) sum += (double)A[m * lda + k] * (double)w[k];
          r = (float)sum;
        } else {
          float sum = 0.0f;
          for (size_t k = 0; k < K; ++k) {
            float p = A[m * lda + k] * w[k];
            sum += p;
          }
          r = sum;
        }
        float dv = (fusion_type == 2 && D) ? D[m * ldd + n] : 0.0f;
        C[m * ldc + n] = orc_epilogue(r, fusion_type, fusion_op, dv);
      }
    }
    free(w);
  }
}

/* Fast CPU baseline of the same contraction: dequantise a row once, then a
 * vectorisable float dot per activation row.  Same arithmetic as acc64 = 0
 * up to summation order; used only as the timed CPU arm. */
__attribute__((target_clones("avx2", "default")))
ORC_API void orc_qmatmul_blocks_fast(int fmt, const float *A, const uint8_t *W, float *C, size_t M,
                                     size_t K, size_t N, size_t lda, size_t ldc) {
  size_t rb = orc_row_bytes(fmt, K);
#pragma omp parallel
  {
    float *w = (float *)malloc(sizeof(float) * (K + 256));
#pragma omp for schedule(static)
    for (long nn = 0; nn < (long)N; ++nn) {
      size_t n = (size_t)nn;
      orc_dequant(fmt, W + n * rb, w, K);
      for (size_t m = 0; m < M; ++m) {
        const float *a = A + m * lda;
        float s0 = 0, s1 = 0, s2 = 0, s3 = 0, s4 = 0, s5 = 0, s6 = 0, s7 = 0;
        size_t k = 0;
        for (; k + 8 <= K; k += 8) {
          s0 += a[k] * w[k];
          s1 += a[k + 1] * w[k + 1];
          s2 += a[k + 2] * w[k + 2];
          s3 += a[k + 3] * w[k + 3];
          s4 += a[k + 4] * w[k + 4];
          s5 += a[k + 5] * w[k + 5];
          s6 += a[k + 6] * w[k + 6];
          s7 += a[k + 7] * w[k + 7];
        }
        for (; k < K; ++k) s0 += a[k] * w[k];
        C[m * ldc + n] = ((s0 + s1) + (s2 + s3)) + ((s4 + s5) + (s6 + s7));
      }
    }
    free(w);
  }
}

/* Dense float contraction C[M,N] = A[M,K] * Wf[N,K]^T on already dequantised
 * weights: the scalar loop of the reference's tests (tests/harness/OpRegistry.h:2043-2050
 * float accumulator; tests/runtime/RuntimeTests.cpp:2907-2920 double accumulator),
 * output rows spread over the OpenMP threads. */
ORC_API void orc_matmul_dense(const float *A, const float *Wf, float *C, size_t M, size_t K, size_t N,
                              size_t lda, size_t ldw, size_t ldc, int acc64) {
#pragma omp parallel for schedule(static)
  for (long nn = 0; nn < (long)N; ++nn) {
    const float *w = Wf + (size_t)nn * ldw;
    for (size_t m = 0; m < M; ++m) {
      const float *a = A + m * lda;
      if (acc64) {
        double sum = 0.0;
        for (size_t k = 0; k < K; ++k) sum += (double)a[k] * (double)w[k];
        C[m * ldc + (size_t)nn] = (float)sum;
      } else {
        float sum = 0.0f;
        for (size_t k = 0; k < K; ++k) sum += a[k] * w[k];
        C[m * ldc + (size_t)nn] = sum;
      }
    }
  }
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* First steps past the matmul path: the producer / consumers of its operands  */
/* in a decoder layer.                                                        */
/* ------------------------------------------------------------------------- */

/* operators/impl/rmsnorm/RMSNorm.cu:6-37 -- y = x * rsqrt(mean(x^2) + eps) * weight per row of
 * `dim` floats (row stride ldx); the sum of squares is accumulated in double here, so the
 * checker is the more exact side of a tolerance comparison. */
ORC_API void orc_rmsnorm(const float *x, const float *weight, float *y, size_t rows, size_t dim, size_t ldx, float eps) {
  for (size_t r = 0; r < rows; ++r) {
    const float *xr = x + r * ldx;
    double ss = 0.0;
    for (size_t i = 0; i < dim; ++i) ss += (double)xr[i] * (double)xr[i];
    double scale = 1.0 / sqrt(ss / (double)dim + (double)eps);
    for (size_t i = 0; i < dim; ++i) y[r * ldx + i] = (float)((double)xr[i] * scale * (double)weight[i]);
  }
}

/* operators/impl/memory/Embedding.cu:18-35 -- out[i, :] = table[indices[i], :], rows padded to 4 floats. */
ORC_API void orc_embedding(const uint32_t *indices, const float *table, float *out, size_t n, size_t dim) {
  size_t ld = (dim + 3) & ~(size_t)3;
  for (size_t i = 0; i < n; ++i) memcpy(out + i * ld, table + (size_t)indices[i] * ld, ld * sizeof(float));
}

/* operators/impl/memory/EmbeddingCol.cu:16-44 -- column gather out[i, d] = M[d, indices[i]] from a
 * [dim, vocab] matrix: format 0 fp16 (raw bits), format 1 int8 values times the fp16 scale of the
 * 32-row group, scales [dim / 32, scale_stride]. */
ORC_API void orc_embedding_col(int format, const uint32_t *indices, const void *matrix, const uint16_t *scales, float *out,
                               size_t n, size_t dim, size_t vocab_stride, size_t scale_stride, size_t out_stride) {
  for (size_t i = 0; i < n; ++i)
    for (size_t d = 0; d < dim; ++d) {
      size_t idx = d * vocab_stride + indices[i];
      float v;
      if (format == 0)
        v = orc_f16_to_f32(((const uint16_t *)matrix)[idx]);
      else
        v = (float)((const int8_t *)matrix)[idx] * orc_f16_to_f32(scales[(d >> 5) * scale_stride + indices[i]]);
      out[i * out_stride + d] = v;
    }
}

/* operators/impl/reduce/ReduceArg.cu:27-59 -- arg-max / arg-min with the reference's tie rule:
 * 256 threads scan i = t, t + 256, ... keeping the FIRST strictly better value, then a
 * shared-memory tree (strides 128 .. 1) keeps the lower position on ties; both steps are replayed
 * here literally.  (Among equal extremes that prefers the smallest bit-reversed i % 256, then the
 * smallest i.)  The result is returned as a float. */
ORC_API float orc_argreduce(const float *v, size_t n, int is_max) {
  float best[256];
  uint32_t idx[256];
  for (int t = 0; t < 256; ++t) {
    best[t] = is_max ? -3.402823466e+38f : 3.402823466e+38f;
    idx[t] = 0;
    for (size_t i = (size_t)t; i < n; i += 256)
      if (is_max ? v[i] > best[t] : v[i] < best[t]) {
        best[t] = v[i];
        idx[t] = (uint32_t)i;
      }
  }
  for (int stride = 128; stride > 0; stride >>= 1)
    for (int t = 0; t < stride; ++t)
      if (is_max ? best[t + stride] > best[t] : best[t + stride] < best[t]) {
        best[t] = best[t + stride];
        idx[t] = idx[t + stride];
      }
  return (float)idx[0];
}

/* IEEE round-to-nearest-even float -> half (the conversion the device's __float2half performs
 * when the reference's fp16 cache variants store a value, AttentionCommon.cuh:18-20). */
ORC_API uint16_t orc_f32_to_f16_rne(float v) {
  uint32_t u;
  memcpy(&u, &v, sizeof(u));
  uint32_t sign = (u >> 16) & 0x8000u, mag = u & 0x7FFFFFFFu;
  if (mag >= 0x7F800000u) return (uint16_t)(sign | (mag > 0x7F800000u ? 0x7E00u : 0x7C00u));
  if (mag >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520: infinity */
  if (mag < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25: zero (a tie goes to even) */
  int32_t e = (int32_t)(mag >> 23) - 127;
  uint32_t m = (mag & 0x7FFFFFu) | 0x800000u;
  uint32_t shift = e < -14 ? (uint32_t)(13 + (-14 - e)) : 13u; /* subnormal halves drop more bits */
  uint32_t kept = m >> shift, rem = m & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (kept & 1u))) ++kept;
  if (e < -14) return (uint16_t)(sign | kept); /* a carry into bit 10 is the smallest normal */
  return (uint16_t)(sign | ((((uint32_t)(e + 15)) << 10) + (kept - 0x400u)));
}

/* operators/impl/attention/FusedRoPEKVWrite.cu:13-75 -- half-split rotary embedding of q and k
 * at position pos (tables [max_seq][head_dim / 2]), roped k and v written to row pos of the
 * caches (row stride ld; kv_half: caches hold halves, stored round-to-nearest-even).  Plain
 * float products and sums in the kernel's order. */
ORC_API void orc_rope_kv_write(int kv_half, const float *q, const float *k, const float *v, uint32_t pos, const float *cos_t,
                               const float *sin_t, void *k_cache, void *v_cache, float *q_out, size_t q_dim, size_t kv_dim,
                               size_t head_dim, size_t ld) {
  size_t half = head_dim / 2;
  const float *c = cos_t + (size_t)pos * half, *s = sin_t + (size_t)pos * half;
  for (size_t pass = 0; pass < 2; ++pass) {
    const float *x = pass ? k : q;
    size_t n = pass ? kv_dim : q_dim;
    for (size_t i = 0; i < n; ++i) {
      size_t in_head = i % head_dim;
      volatile float a, b; /* keep the two products rounded separately */
      float r;
      if (in_head < half) {
        a = x[i] * c[in_head];
        b = x[i + half] * s[in_head];
        r = a - b;
      } else {
        a = x[i - half] * s[in_head - half];
        b = x[i] * c[in_head - half];
        r = a + b;
      }
      if (!pass) q_out[i] = r;
      else if (kv_half) ((uint16_t *)k_cache)[(size_t)pos * ld + i] = orc_f32_to_f16_rne(r);
      else ((float *)k_cache)[(size_t)pos * ld + i] = r;
    }
  }
  for (size_t i = 0; i < kv_dim; ++i) {
    if (kv_half) ((uint16_t *)v_cache)[(size_t)pos * ld + i] = orc_f32_to_f16_rne(v[i]);
    else ((float *)v_cache)[(size_t)pos * ld + i] = v[i];
  }
}

/* operators/impl/attention/Attention.cu:31-108 (and the CPU helper of the reference's own test,
 * tests/runtime/RuntimeTests.cpp:5946-5991) -- per query head: scores = (q . K[t]) * scale over
 * the first seq_len cache rows, softmax, weighted sum of V; head h reads KV head
 * h / (n_heads / n_kv_heads).  Accumulated in double, so the checker is the more exact side. */
ORC_API void orc_attention(int kv_half, const float *q, const void *k_cache, const void *v_cache, size_t seq_len, float *out,
                           size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t ld, float scale) {
  size_t n_rep = n_heads / n_kv_heads;
  double *score = (double *)malloc((seq_len ? seq_len : 1) * sizeof(double));
  for (size_t h = 0; h < n_heads; ++h) {
    size_t kvh = h / n_rep;
    double mx = -1e30, sum = 0.0;
    for (size_t t = 0; t < seq_len; ++t) {
      double dot = 0.0;
      for (size_t d = 0; d < head_dim; ++d) {
        size_t at = t * ld + kvh * head_dim + d;
        double kv = kv_half ? (double)orc_f16_to_f32(((const uint16_t *)k_cache)[at]) : (double)((const float *)k_cache)[at];
        dot += (double)q[h * head_dim + d] * kv;
      }
      score[t] = dot * (double)scale;
      if (score[t] > mx) mx = score[t];
    }
    for (size_t t = 0; t < seq_len; ++t) {
      score[t] = exp(score[t] - mx);
      sum += score[t];
    }
    for (size_t d = 0; d < head_dim; ++d) {
      double acc = 0.0;
      for (size_t t = 0; t < seq_len; ++t) {
        size_t at = t * ld + kvh * head_dim + d;
        double vv = kv_half ? (double)orc_f16_to_f32(((const uint16_t *)v_cache)[at]) : (double)((const float *)v_cache)[at];
        acc += score[t] * vv;
      }
      out[h * head_dim + d] = seq_len ? (float)(acc / sum) : 0.0f;
    }
  }
  free(score);
}

