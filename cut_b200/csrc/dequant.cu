// Raw GGUF blocks -> fp32 [rows, ldo], bit-exact with the reference.
//
// Replaces the reference's dequant kernels (operators/impl/dequant/DequantQ4K.cu:6-50,
// DequantQ5K.cu, DequantQ6K.cu, DequantBF16.cu, helpers DequantCommon.cuh:16-70) and
// adds the Q8_0 / Q4_0 / Q4_1 / Q5_0 cases the reference only has on the CPU
// (interface/loader/gguf/gguf_reader.cpp:541-660, 826-850).  Every format follows the
// loader's dequantiser operation by operation (each product and the subtract rounded on
// their own), so the output equals its float32 bits.
//
// The op is write-bound (4 bytes out per 0.56-1.06 bytes in).  Each thread
// decodes 8 consecutive weights of one block -- the block header is read once
// per thread through the read-only path instead of once per element -- and
// stores them as two 16-byte vectors, so a warp writes 1 KB of contiguous
// output per instruction pair.  Grid = a multiple of the SM count, grid-stride.
#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

__device__ __forceinline__ uint32_t ldg8(const uint8_t *p) { return __ldg(p); }
__device__ __forceinline__ uint32_t ldg16(const uint8_t *p) { return ldg8(p) | (ldg8(p + 1) << 8); }
// 32-bit little-endian read at any byte alignment
__device__ __forceinline__ uint32_t ldg32u(const uint8_t *p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  if ((a & 3) == 0) return __ldg(reinterpret_cast<const uint32_t *>(p));
  if ((a & 1) == 0) {
    const uint16_t *q = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t)__ldg(q) | ((uint32_t)__ldg(q + 1) << 16);
  }
  return ldg8(p) | (ldg8(p + 1) << 8) | (ldg8(p + 2) << 16) | (ldg8(p + 3) << 24);
}

// 6-bit (scale, min) of sub-block j from the 12 packed bytes of a Q4_K / Q5_K super-block
// (gguf_reader.cpp:668-676).
__device__ __forceinline__ uint32_t ldg32a(const uint8_t *p) { return __ldg(reinterpret_cast<const uint32_t *>(p)); }  // 4-byte aligned

__device__ __forceinline__ void scale_min_k4(const uint8_t *sc, uint32_t j, uint32_t &s, uint32_t &m) {
  // the 12 bytes as three words (bytes 0-3: low scales, 4-7: low mins, 8-11: high nibbles);
  // Q4_K / Q5_K super-blocks are 4-byte aligned (checked at launch)
  const uint32_t w0 = ldg32a(sc), w1 = ldg32a(sc + 4), w2 = ldg32a(sc + 8);
  const uint32_t sh = 8 * (j & 3);
  const uint32_t a = (w0 >> sh) & 0xFF, b = (w1 >> sh) & 0xFF, c = (w2 >> sh) & 0xFF;
  if (j < 4) {
    s = a & 63;
    m = b & 63;
  } else {
    s = (c & 0xF) | ((a >> 6) << 4);
    m = (c >> 4) | ((b >> 6) << 4);
  }
}

// 8 weights [8*oct, 8*oct+8) of the 32-weight (Q8_0, Q4_0) or 256-weight (Q4_K, Q5_K,
// Q6_K) block at `b`; for BF16 `b` points at the first of `valid` (<= 8) elements.
template <int FMT> __device__ __forceinline__ void decode8(const uint8_t *b, uint32_t oct, float (&v)[8], uint32_t valid) {
  if constexpr (FMT == CUTB_BF16) {
    // the upper half of a float32 (gguf_reader.cpp:860-870, DequantBF16.cu:20-28)
    if (valid >= 8 && (reinterpret_cast<uintptr_t>(b) & 15) == 0) {
      const uint4 w = __ldg(reinterpret_cast<const uint4 *>(b));
      const uint32_t x[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(x[i] << 16);
        v[2 * i + 1] = __uint_as_float(x[i] & 0xFFFF0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = (uint32_t)i < valid ? __uint_as_float(ldg16(b + 2 * i) << 16) : 0.f;
    }
  } else if constexpr (FMT == CUTB_Q5_K) {
    // gguf_reader.cpp:726-772: group g of 64 = sub-blocks 2g (low nibbles) and 2g + 1 (high
    // nibbles) of the group's 32 ql bytes; bit j of qh[l] is element l's fifth bit in sub-block j
    const uint32_t j = oct >> 2, l0 = (oct & 3) * 8;
    const uint32_t hdr = ldg32a(b);
    const float d = h2f_bits(hdr & 0xFFFF), dmin = h2f_bits(hdr >> 16);
    uint32_t s, m;
    scale_min_k4(b + 4, j, s, m);
    const float d1 = __fmul_rn(d, (float)s), dm = __fmul_rn(dmin, (float)m);
    const uint8_t *ql = b + 48 + (j >> 1) * 32 + l0, *qh = b + 16 + l0;
    const uint32_t sh = (j & 1) * 4;
    const uint32_t w[2] = {ldg32a(ql), ldg32a(ql + 4)}, h[2] = {ldg32a(qh), ldg32a(qh + 4)};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t q = ((w[i >> 2] >> (8 * (i & 3) + sh)) & 0xF) + (((h[i >> 2] >> (8 * (i & 3) + j)) & 1) << 4);
      v[i] = __fsub_rn(__fmul_rn(d1, (float)q), dm);
    }
  } else if constexpr (FMT == CUTB_Q6_K) {
    // gguf_reader.cpp:774-824: half (128 elements), run r of 32, element l of the run
    const uint32_t half = oct >> 4, r = (oct >> 2) & 3, l0 = (oct & 3) * 8;
    const float d = h2f_bits(ldg16(b + 208));
    const uint8_t *ql = b + 64 * half + 32 * (r & 1) + l0, *qh = b + 128 + 32 * half + l0;
    const int sc = (int)(int8_t)ldg8(b + 192 + 8 * half + 2 * r + (l0 >> 4));
    const float ds = __fmul_rn(d, (float)sc);
    const uint32_t sh = (r >> 1) * 4;
    const uint32_t w[2] = {ldg32u(ql), ldg32u(ql + 4)}, h[2] = {ldg32u(qh), ldg32u(qh + 4)};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = (int)(((w[i >> 2] >> (8 * (i & 3) + sh)) & 0xF) | (((h[i >> 2] >> (8 * (i & 3) + 2 * r)) & 3) << 4)) - 32;
      v[i] = __fmul_rn(ds, (float)q);
    }
  } else if constexpr (FMT == CUTB_Q8_0) {
    const float d = h2f_bits(ldg16(b));
    const uint32_t w0 = ldg32u(b + 2 + 8 * oct), w1 = ldg32u(b + 6 + 8 * oct);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = (float)(int8_t)((w0 >> (8 * i)) & 0xFF) * d;
      v[4 + i] = (float)(int8_t)((w1 >> (8 * i)) & 0xFF) * d;
    }
  } else if constexpr (FMT == CUTB_Q4_1) {
    // gguf_reader.cpp:574-611: value = float(nibble) * d + m, the product and the sum rounded on their own
    const float d = h2f_bits(ldg16(b)), m = h2f_bits(ldg16(b + 2));
    const uint32_t sh = (oct >> 1) * 4;
    const uint32_t w0 = ldg32u(b + 4 + 8 * (oct & 1)), w1 = ldg32u(b + 8 + 8 * (oct & 1));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = __fadd_rn(__fmul_rn((float)((w0 >> (8 * i + sh)) & 0xF), d), m);
      v[4 + i] = __fadd_rn(__fmul_rn((float)((w1 >> (8 * i + sh)) & 0xF), d), m);
    }
  } else if constexpr (FMT == CUTB_Q5_0) {
    // gguf_reader.cpp:613-660: nibbles as Q4_0, bit e of qh is element e's fifth bit; value = float(q5 - 16) * d
    const float d = h2f_bits(ldg16(b));
    const uint32_t qh = ldg16(b + 2) | (ldg16(b + 4) << 16);
    const uint32_t sh = (oct >> 1) * 4, e0 = 8 * oct;
    const uint32_t w0 = ldg32u(b + 6 + 8 * (oct & 1)), w1 = ldg32u(b + 10 + 8 * (oct & 1));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int q0 = (int)(((w0 >> (8 * i + sh)) & 0xF) | (((qh >> (e0 + i)) & 1u) << 4)) - 16;
      const int q1 = (int)(((w1 >> (8 * i + sh)) & 0xF) | (((qh >> (e0 + 4 + i)) & 1u) << 4)) - 16;
      v[i] = (float)q0 * d;
      v[4 + i] = (float)q1 * d;
    }
  } else if constexpr (FMT == CUTB_Q4_0) {
    const float d = h2f_bits(ldg16(b));
    // elements 8*oct.. live in bytes (8*oct & 15).. ; low nibbles for oct < 2, high for oct >= 2
    const uint32_t sh = (oct >> 1) * 4;
    const uint32_t w0 = ldg32u(b + 2 + 8 * (oct & 1)), w1 = ldg32u(b + 6 + 8 * (oct & 1));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = (float)((int)((w0 >> (8 * i + sh)) & 0xF) - 8) * d;
      v[4 + i] = (float)((int)((w1 >> (8 * i + sh)) & 0xF) - 8) * d;
    }
  } else {
    const uint32_t j = oct >> 2, l0 = (oct & 3) * 8;  // sub-block, first element inside it
    const uint32_t hdr = __ldg(reinterpret_cast<const uint32_t *>(b));
    const float d = h2f_bits(hdr & 0xFFFF), dmin = h2f_bits(hdr >> 16);
    uint32_t s, m;
    scale_min_k4(b + 4, j, s, m);
    // value = (d * sc) * q - dmin * m, each product rounded on its own
    // (gguf_reader.cpp:700-718, DequantQ4K.cu:39-46); both products are exact.
    const float d1 = __fmul_rn(d, (float)s), dm = __fmul_rn(dmin, (float)m);
    const uint8_t *q = b + 16 + (j >> 1) * 32 + l0;
    const uint32_t sh = (j & 1) * 4;
    const uint32_t w0 = __ldg(reinterpret_cast<const uint32_t *>(q)), w1 = __ldg(reinterpret_cast<const uint32_t *>(q + 4));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = __fsub_rn(__fmul_rn(d1, (float)((w0 >> (8 * i + sh)) & 0xF)), dm);
      v[4 + i] = __fsub_rn(__fmul_rn(d1, (float)((w1 >> (8 * i + sh)) & 0xF)), dm);
    }
  }
}

template <int FMT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t *__restrict__ raw, float *__restrict__ out, uint32_t rows,
                                                      uint32_t cols, uint32_t ldo, uint64_t row_bytes_, int vec_ok) {
  constexpr uint32_t BE = block_elems(FMT), BB = block_bytes(FMT);
  const uint32_t octs_per_row = (cols + 7) / 8;
  // grid.x walks a row's groups of eight weights, grid.y the rows: no division per element
  for (uint32_t r = blockIdx.y; r < rows; r += gridDim.y)
  for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < octs_per_row; o += gridDim.x * blockDim.x) {
    const uint32_t k = o * 8;
    const uint8_t *b = raw + (uint64_t)r * row_bytes_ + (uint64_t)(k / BE) * BB;
    float v[8];
    decode8<FMT>(b, (k % BE) / 8, v, cols - k);
    float *dst = out + (uint64_t)r * ldo + k;
    if (vec_ok && k + 8 <= cols) {
      // written once, read by another kernel much later: streaming stores keep them from
      // displacing the raw blocks in L2
      __stcs(reinterpret_cast<float4 *>(dst), make_float4(v[0], v[1], v[2], v[3]));
      __stcs(reinterpret_cast<float4 *>(dst) + 1, make_float4(v[4], v[5], v[6], v[7]));
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (k + e < cols) dst[e] = v[e];
    }
  }
}

// Row gather with dequantisation: out[i, :] = dequant(row indices[i]) -- the embedding lookup when the
// (tied) table is kept as raw GGUF blocks, one row per token.  A row index >= rows writes zeros and
// reports through *status.
template <int FMT>
__global__ void __launch_bounds__(256) dequant_gather_kernel(const uint32_t *__restrict__ indices, const uint8_t *__restrict__ raw,
                                                             float *__restrict__ out, uint32_t n, uint32_t rows, uint32_t cols,
                                                             uint32_t ldo, uint64_t row_bytes_, int vec_ok, int *status) {
  constexpr uint32_t BE = block_elems(FMT), BB = block_bytes(FMT);
  const uint32_t octs_per_row = (cols + 7) / 8;
  for (uint32_t i = blockIdx.y; i < n; i += gridDim.y) {
    const uint32_t r = __ldg(indices + i);
    if (r >= rows && threadIdx.x == 0 && blockIdx.x == 0 && status) atomicExch(status, (int)CUTB_ERR_INVALID);
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < octs_per_row; o += gridDim.x * blockDim.x) {
      const uint32_t k = o * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (r < rows) decode8<FMT>(raw + (uint64_t)r * row_bytes_ + (uint64_t)(k / BE) * BB, (k % BE) / 8, v, cols - k);
      float *dst = out + (uint64_t)i * ldo + k;
      if (vec_ok && k + 8 <= cols) {
        *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *(reinterpret_cast<float4 *>(dst) + 1) = make_float4(v[4], v[5], v[6], v[7]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (k + e < cols) dst[e] = v[e];
      }
    }
  }
}

// Any dequantisable block format -> Q8_0 GGUF blocks, on the device: the runner's load-time requantisation
// of the formats its matmul does not take (interface/runner/llama/llama.cpp:750-767 with quantizeRowsQ8_0,
// :488-505), fused with the dequantisation.  One thread per group of 32 weights: exact dequantised values
// (as cutb_dequant), d = amax / 127 stored through the runner's float -> half, q = lround(x * (1 / d)).
template <int FMT>
__global__ void __launch_bounds__(256) requant_q8_0_blocks_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ out,
                                                                  uint64_t rows, uint32_t cols, uint64_t row_bytes_) {
  constexpr uint32_t BE = block_elems(FMT), BB = block_bytes(FMT);
  const uint64_t groups_per_row = cols / 32, total = rows * groups_per_row;
  for (uint64_t gidx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; gidx < total; gidx += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t r = gidx / groups_per_row;
    const uint32_t k = (uint32_t)(gidx % groups_per_row) * 32;
    const uint8_t *b = raw + r * row_bytes_ + (uint64_t)(k / BE) * BB;
    float v[32];
#pragma unroll
    for (int o = 0; o < 4; ++o) {
      float t8[8];
      decode8<FMT>(FMT == CUTB_BF16 ? raw + r * row_bytes_ + (uint64_t)(k + 8 * o) * 2 : b, (k % BE) / 8 + o, t8, 8);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[8 * o + e] = t8[e];
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    uint16_t *o16 = reinterpret_cast<uint16_t *>(out + gidx * 34);  // 34-byte blocks: 2-byte aligned
    o16[0] = f32_to_f16_runner(d);
#pragma unroll
    for (int w = 0; w < 16; ++w) {
      // lroundf: nearest, halves away from zero; the product is rounded to float first, as on the CPU
      const int q0 = (int)(int8_t)lroundf(__fmul_rn(v[2 * w], id)), q1 = (int)(int8_t)lroundf(__fmul_rn(v[2 * w + 1], id));
      o16[1 + w] = (uint16_t)(((uint32_t)q0 & 0xFFu) | (((uint32_t)q1 & 0xFFu) << 8));
    }
  }
}

}  // namespace

int requant_q8_0_blocks_launch(int format, const void *raw, void *out, uint64_t rows, uint32_t cols, cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  const uint64_t total = rows * (cols / 32);
  if (total == 0) return CUTB_OK;
  if ((format == CUTB_Q4_K || format == CUTB_Q5_K) && (reinterpret_cast<uintptr_t>(raw) % 4 != 0)) {
    set_last_error("requant_q8_0_blocks: Q4_K / Q5_K blocks must be 4-byte aligned");
    return CUTB_ERR_INVALID;
  }
  uint64_t blocks = (total + 255) / 256;
  if (blocks > (uint64_t)di.sm_count * 16) blocks = (uint64_t)di.sm_count * 16;
  const unsigned g = (unsigned)blocks;
  const uint8_t *r = reinterpret_cast<const uint8_t *>(raw);
  uint8_t *o = reinterpret_cast<uint8_t *>(out);
  const uint64_t rb = row_bytes(format, cols);
  switch (format) {
    case CUTB_Q8_0: requant_q8_0_blocks_kernel<CUTB_Q8_0><<<g, 256, 0, stream>>>(r, o, rows, cols, rb); break;
    case CUTB_Q4_0: requant_q8_0_blocks_kernel<CUTB_Q4_0><<<g, 256, 0, stream>>>(r, o, rows, cols, rb); break;
    case CUTB_Q5_K: requant_q8_0_blocks_kernel<CUTB_Q5_K><<<g, 256, 0, stream>>>(r, o, rows, cols, rb); break;
    case CUTB_Q6_K: requant_q8_0_blocks_kernel<CUTB_Q6_K><<<g, 256, 0, stream>>>(r, o, rows, cols, rb); break;
    case CUTB_BF16: requant_q8_0_blocks_kernel<CUTB_BF16><<<g, 256, 0, stream>>>(r, o, rows, cols, rb); break;
    case CUTB_Q4_1: requant_q8_0_blocks_kernel<CUTB_Q4_1><<<g, 256, 0, stream>>>(r, o, rows, cols, rb); break;
    case CUTB_Q5_0: requant_q8_0_blocks_kernel<CUTB_Q5_0><<<g, 256, 0, stream>>>(r, o, rows, cols, rb); break;
    default: requant_q8_0_blocks_kernel<CUTB_Q4_K><<<g, 256, 0, stream>>>(r, o, rows, cols, rb); break;
  }
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

int dequant_gather_launch(int format, const uint32_t *indices, const void *raw, float *out, uint32_t n, uint32_t rows, uint32_t cols,
                          uint32_t ldo, int *status, cudaStream_t stream) {
  if (n == 0 || cols == 0) return CUTB_OK;
  if ((format == CUTB_Q4_K || format == CUTB_Q5_K) && (reinterpret_cast<uintptr_t>(raw) % 4 != 0)) {
    set_last_error("embedding_blocks: Q4_K / Q5_K blocks must be 4-byte aligned");
    return CUTB_ERR_INVALID;
  }
  if ((format == CUTB_Q4_K || format == CUTB_Q5_K || format == CUTB_Q6_K) && cols % 256 != 0) {
    set_last_error("embedding_blocks: K-quant rows are whole 256-weight super-blocks, cols = %u", cols);
    return CUTB_ERR_INVALID;
  }
  if (format == CUTB_BF16 && (reinterpret_cast<uintptr_t>(raw) % 2 != 0)) {
    set_last_error("embedding_blocks: BF16 input must be 2-byte aligned");
    return CUTB_ERR_INVALID;
  }
  uint32_t gx = ((cols + 7) / 8 + 255) / 256;
  if (gx > 64) gx = 64;
  const dim3 g(gx, n < 65535u ? n : 65535u);
  const int vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (ldo % 4 == 0);
  const uint8_t *r = reinterpret_cast<const uint8_t *>(raw);
  const uint64_t rb = row_bytes(format, cols);
  switch (format) {
    case CUTB_Q8_0: dequant_gather_kernel<CUTB_Q8_0><<<g, 256, 0, stream>>>(indices, r, out, n, rows, cols, ldo, rb, vec_ok, status); break;
    case CUTB_Q4_0: dequant_gather_kernel<CUTB_Q4_0><<<g, 256, 0, stream>>>(indices, r, out, n, rows, cols, ldo, rb, vec_ok, status); break;
    case CUTB_Q5_K: dequant_gather_kernel<CUTB_Q5_K><<<g, 256, 0, stream>>>(indices, r, out, n, rows, cols, ldo, rb, vec_ok, status); break;
    case CUTB_Q6_K: dequant_gather_kernel<CUTB_Q6_K><<<g, 256, 0, stream>>>(indices, r, out, n, rows, cols, ldo, rb, vec_ok, status); break;
    case CUTB_BF16: dequant_gather_kernel<CUTB_BF16><<<g, 256, 0, stream>>>(indices, r, out, n, rows, cols, ldo, rb, vec_ok, status); break;
    case CUTB_Q4_1: dequant_gather_kernel<CUTB_Q4_1><<<g, 256, 0, stream>>>(indices, r, out, n, rows, cols, ldo, rb, vec_ok, status); break;
    case CUTB_Q5_0: dequant_gather_kernel<CUTB_Q5_0><<<g, 256, 0, stream>>>(indices, r, out, n, rows, cols, ldo, rb, vec_ok, status); break;
    default: dequant_gather_kernel<CUTB_Q4_K><<<g, 256, 0, stream>>>(indices, r, out, n, rows, cols, ldo, rb, vec_ok, status); break;
  }
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

int dequant_launch(int format, const void *raw, float *out, uint32_t rows, uint32_t cols, uint32_t ldo,
                   cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  const uint64_t total = (uint64_t)rows * ((cols + 7) / 8);
  if (total == 0) return CUTB_OK;
  // about 8 CTAs per SM in all: enough along a row to cover it once, the rest along the rows
  const uint32_t cap = (uint32_t)di.sm_count * 8;
  uint32_t gx = ((cols + 7) / 8 + 255) / 256;
  if (gx > cap) gx = cap;
  uint32_t gy = cap / gx;
  if (gy > rows) gy = rows;
  if (gy > 65535u) gy = 65535u;
  if (gy == 0) gy = 1;
  const dim3 blocks(gx, gy);
  const int vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (ldo % 4 == 0);
  const uint8_t *r = reinterpret_cast<const uint8_t *>(raw);
  const uint64_t rb = row_bytes(format, cols);
  if ((format == CUTB_Q4_K || format == CUTB_Q5_K) && (reinterpret_cast<uintptr_t>(raw) % 4 != 0)) {
    set_last_error("dequant: Q4_K / Q5_K blocks must be 4-byte aligned");
    return CUTB_ERR_INVALID;
  }
  if ((format == CUTB_Q5_K || format == CUTB_Q6_K) && cols % 256 != 0) {
    set_last_error("dequant: Q5_K / Q6_K rows are whole 256-weight super-blocks, cols = %u", cols);
    return CUTB_ERR_INVALID;
  }
  if (format == CUTB_BF16 && (reinterpret_cast<uintptr_t>(raw) % 2 != 0)) {
    set_last_error("dequant: BF16 input must be 2-byte aligned");
    return CUTB_ERR_INVALID;
  }
  const dim3 g = blocks;
  switch (format) {
    case CUTB_Q8_0: dequant_kernel<CUTB_Q8_0><<<g, 256, 0, stream>>>(r, out, rows, cols, ldo, rb, vec_ok); break;
    case CUTB_Q4_0: dequant_kernel<CUTB_Q4_0><<<g, 256, 0, stream>>>(r, out, rows, cols, ldo, rb, vec_ok); break;
    case CUTB_Q5_K: dequant_kernel<CUTB_Q5_K><<<g, 256, 0, stream>>>(r, out, rows, cols, ldo, rb, vec_ok); break;
    case CUTB_Q6_K: dequant_kernel<CUTB_Q6_K><<<g, 256, 0, stream>>>(r, out, rows, cols, ldo, rb, vec_ok); break;
    case CUTB_BF16: dequant_kernel<CUTB_BF16><<<g, 256, 0, stream>>>(r, out, rows, cols, ldo, rb, vec_ok); break;
    case CUTB_Q4_1: dequant_kernel<CUTB_Q4_1><<<g, 256, 0, stream>>>(r, out, rows, cols, ldo, rb, vec_ok); break;
    case CUTB_Q5_0: dequant_kernel<CUTB_Q5_0><<<g, 256, 0, stream>>>(r, out, rows, cols, ldo, rb, vec_ok); break;
    default: dequant_kernel<CUTB_Q4_K><<<g, 256, 0, stream>>>(r, out, rows, cols, ldo, rb, vec_ok); break;
  }
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace cutb
