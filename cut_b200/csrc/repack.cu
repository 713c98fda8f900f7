// Load-time repacks of GGUF tensors on the device, bit-exact with the CPU code they replace.
//
// The reference builds its matmul operands on the CPU: the loader splits Q8_0 / Q4_0 blocks
// into a value plane and a scale plane (interface/loader/gguf/gguf_reader.cpp:389-501), the
// runner transposes them into the [K, N] orientation, re-encodes Q4_K super-blocks as affine
// 4-bit planes (interface/runner/llama/llama.cpp:573-619) and requantises other types to Q8_0
// (llama.cpp:488-505), all single-threaded and with a scalar read-modify-write per nibble.
// The block kernels of this library consume raw GGUF bytes and need none of it; these kernels
// exist for callers that keep the reference's plane layout: upload the raw tensor once, derive
// the planes here.  Byte and integer work is exact by construction; the two float -> half
// conversions follow the runner's own rounding (round half up on the dropped bits, not
// ties-to-even: llama.cpp:445-482).
#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

__device__ __forceinline__ uint32_t ld8(const uint8_t *p) { return __ldg(p); }
__device__ __forceinline__ uint32_t ld16(const uint8_t *p) { return ld8(p) | (ld8(p + 1) << 8); }

// gguf_reader.cpp:389-501: block b of a row-major [rows, cols] tensor -> 32 int8 (Q8_0) or 16
// packed bytes (Q4_0) at their place in the value plane, and the block's f16 scale.  One thread
// per 2 bytes of a block's payload: consecutive threads write consecutive bytes.
template <int FMT>
__global__ void __launch_bounds__(256) separate_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ values,
                                                       uint16_t *__restrict__ scales, uint64_t nblocks) {
  constexpr uint32_t BB = FMT == CUTB_Q8_0 ? 34u : 18u, PB = BB - 2;  // block bytes, payload bytes
  constexpr uint32_t TPB = PB / 2;                                    // threads per block of weights
  const uint64_t total = nblocks * TPB;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t b = i / TPB;
    const uint32_t t = (uint32_t)(i % TPB);
    const uint8_t *p = raw + b * BB;  // blocks are 2-byte aligned (BB is even and the tensor base is)
    const uint16_t w = __ldg(reinterpret_cast<const uint16_t *>(p + 2 + 2 * t));
    reinterpret_cast<uint16_t *>(values + b * PB)[t] = w;
    if (t == 0) scales[b] = __ldg(reinterpret_cast<const uint16_t *>(p));
  }
}

// out[c * ldo + r] = in[r * ldi + c] for 1- or 2-byte elements, 32 x 32 tiles through shared memory.
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T *__restrict__ in, T *__restrict__ out, uint32_t R, uint32_t C,
                                                        uint64_t ldi, uint64_t ldo) {
  __shared__ T tile[32][33];
  const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const uint32_t c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const uint32_t r = r0 + ty + j, c = c0 + tx;
    if (r < R && c < C) tile[ty + j][tx] = in[(uint64_t)r * ldi + c];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const uint32_t c = c0 + ty + j, r = r0 + tx;
    if (r < R && c < C) out[(uint64_t)c * ldo + r] = tile[tx][ty + j];
  }
}

// llama.cpp:573-619: Q4_K rows -> nibbles [K, N / 2] (low nibble = even n) and f16 planes
// [2 K / 32, N]: rows [0, K / 32) = half(d * sc), rows [K / 32, 2 K / 32) = half(8 d sc - dmin m).
// One thread per (row pair, sub-block of 32 weights): a warp covers 32 consecutive row pairs, so
// its stores of one k are 32 consecutive bytes; the two rows of a pair are combined in registers,
// which removes the reference's read-modify-write per nibble.
__global__ void __launch_bounds__(256) requant_q4k_affine_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ packedT,
                                                                 uint16_t *__restrict__ scalesT, uint32_t N, uint32_t K,
                                                                 uint64_t ldp, uint64_t lds) {
  const uint32_t pairs = N / 2, subs = K / 32, blocksK = K / 32;
  const uint64_t total = (uint64_t)pairs * subs;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t pr = (uint32_t)(i % pairs), sb = (uint32_t)(i / pairs);  // row pair, sub-block along K
    const uint32_t s = sb / 8, j = sb % 8, g = j >> 1, h = j & 1;
    uint32_t q[2][8];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const uint32_t n = 2 * pr + e;
      const uint8_t *blk = raw + ((uint64_t)n * (K / 256) + s) * 144;
      const float d = h2f_bits(ld16(blk)), dmin = h2f_bits(ld16(blk + 2));
      const uint8_t *sc = blk + 4;
      uint32_t scv, mv;
      if (j < 4) {
        scv = ld8(sc + j) & 63;
        mv = ld8(sc + j + 4) & 63;
      } else {
        scv = (ld8(sc + j + 4) & 0xF) | ((ld8(sc + j - 4) >> 6) << 4);
        mv = (ld8(sc + j + 4) >> 4) | ((ld8(sc + j) >> 6) << 4);
      }
      const float scale = __fmul_rn(d, (float)scv);
      const float minv = __fsub_rn(__fmul_rn(8.0f, scale), __fmul_rn(dmin, (float)mv));
      scalesT[(uint64_t)sb * lds + n] = f32_to_f16_runner(scale);
      scalesT[(uint64_t)(blocksK + sb) * lds + n] = f32_to_f16_runner(minv);
      const uint32_t *qs = reinterpret_cast<const uint32_t *>(blk + 16 + g * 32);  // 4-byte aligned: 144 s + 16 + 32 g
#pragma unroll
      for (int w = 0; w < 8; ++w) q[e][w] = (__ldg(qs + w) >> (4 * h)) & 0x0F0F0F0Fu;
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t both = q[0][w] | (q[1][w] << 4);  // four k: byte = nibble(2 pr) | nibble(2 pr + 1) << 4
#pragma unroll
      for (int b = 0; b < 4; ++b) packedT[(uint64_t)(sb * 32 + 4 * w + b) * ldp + pr] = (uint8_t)(both >> (8 * b));
    }
  }
}

// llama.cpp:488-505: float rows -> Q8_0 planes; d = amax / 127 stored through the runner's
// float -> half, q = lround(x * (1 / d)).  One thread per block of 32 values.
__global__ void __launch_bounds__(256) quantize_rows_q8_0_kernel(const float *__restrict__ x, int8_t *__restrict__ values,
                                                                 uint16_t *__restrict__ scales, uint64_t nblocks) {
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (uint64_t)gridDim.x * blockDim.x) {
    const float4 *p = reinterpret_cast<const float4 *>(x + b * 32);
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 f = __ldg(p + i);
      v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    scales[b] = f32_to_f16_runner(d);
    uint32_t packed[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      uint32_t acc = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // lroundf: nearest, halves away from zero; the product is rounded to float first, as on the CPU
        const int qi = (int)(int8_t)lroundf(__fmul_rn(v[4 * w + e], id));
        acc |= ((uint32_t)qi & 0xFFu) << (8 * e);
      }
      packed[w] = acc;
    }
    uint4 *o = reinterpret_cast<uint4 *>(values + b * 32);
    o[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    o[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
  }
}

unsigned grid_for(uint64_t work_items, int sm_count) {
  uint64_t blocks = (work_items + 255) / 256;
  const uint64_t cap = (uint64_t)sm_count * 16;
  if (blocks > cap) blocks = cap;
  return blocks ? (unsigned)blocks : 1u;
}

}  // namespace

int separate_launch(int format, const void *raw, void *values, void *scales, uint64_t rows, uint64_t cols, cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  const uint64_t nblocks = rows * (cols / 32);
  if (nblocks == 0) return CUTB_OK;
  const uint8_t *r = reinterpret_cast<const uint8_t *>(raw);
  if (format == CUTB_Q8_0)
    separate_kernel<CUTB_Q8_0><<<grid_for(nblocks * 16, di.sm_count), 256, 0, stream>>>(
        r, reinterpret_cast<uint8_t *>(values), reinterpret_cast<uint16_t *>(scales), nblocks);
  else
    separate_kernel<CUTB_Q4_0><<<grid_for(nblocks * 8, di.sm_count), 256, 0, stream>>>(
        r, reinterpret_cast<uint8_t *>(values), reinterpret_cast<uint16_t *>(scales), nblocks);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

int transpose_launch(uint32_t elem_bytes, const void *in, void *out, uint32_t R, uint32_t C, uint64_t ldi, uint64_t ldo,
                     cudaStream_t stream) {
  if (R == 0 || C == 0) return CUTB_OK;
  const dim3 grid((C + 31) / 32, (R + 31) / 32);
  if (grid.y > 65535u) {
    set_last_error("transpose: more than 2,097,120 rows");
    return CUTB_ERR_UNSUPPORTED;
  }
  if (elem_bytes == 1)
    transpose_kernel<uint8_t><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint8_t *>(in), reinterpret_cast<uint8_t *>(out), R, C,
                                                        ldi, ldo);
  else
    transpose_kernel<uint16_t><<<grid, 256, 0, stream>>>(reinterpret_cast<const uint16_t *>(in), reinterpret_cast<uint16_t *>(out),
                                                         R, C, ldi, ldo);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

int requant_q4k_affine_launch(const void *raw, void *packedT, void *scalesT, uint32_t N, uint32_t K, uint64_t ldp, uint64_t lds,
                              cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  const uint64_t total = (uint64_t)(N / 2) * (K / 32);
  if (total == 0) return CUTB_OK;
  requant_q4k_affine_kernel<<<grid_for(total, di.sm_count), 256, 0, stream>>>(
      reinterpret_cast<const uint8_t *>(raw), reinterpret_cast<uint8_t *>(packedT), reinterpret_cast<uint16_t *>(scalesT), N, K, ldp,
      lds);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

int quantize_rows_q8_0_launch(const float *x, void *values, void *scales, uint64_t n, cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  const uint64_t nblocks = n / 32;
  if (nblocks == 0) return CUTB_OK;
  quantize_rows_q8_0_kernel<<<grid_for(nblocks, di.sm_count), 256, 0, stream>>>(x, reinterpret_cast<int8_t *>(values),
                                                                               reinterpret_cast<uint16_t *>(scales), nblocks);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace cutb
