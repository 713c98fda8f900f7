// Any-shape quantized matmul, plain SIMT: exact fp32 dequant + fmaf.
//
// Covers everything the specialised kernels do not: odd K / N, unaligned
// buffers, large M on shapes the tensor-core GEMM rejects, and the reference's
// own runtime layout ([K,N] value plane + fp16 scale plane, optional affine
// mins) that its loader and runner hand to MatMulOpNode
// (operators/impl/matmul/MatMulOp.cpp:309-329; element semantics
// MatMulQ4Common.cuh:126-153 and MatMulQ8Common.cuh:127-200).  The dequantised
// weight values are bit-identical to the loader's CPU dequantisers
// (interface/loader/gguf/gguf_reader.cpp:541-572, 678-724, 826-850).
#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

constexpr int GEN_MT = 8;  // activation rows per pass

struct GenParams {
  const uint8_t *W;
  const uint16_t *S;
  const void *A;
  float *C;
  const float *D;
  uint64_t row_bytes;
  uint32_t M, K, N, lda, ldb, lds, ldc, ldd;
  int fusion_type, fusion_op, affine;
};

template <bool AF32> __device__ __forceinline__ float load_a(const void *A, uint64_t i) {
  if constexpr (AF32) return __ldg(reinterpret_cast<const float *>(A) + i);
  return __half2float(__ldg(reinterpret_cast<const __half *>(A) + i));
}

__device__ __forceinline__ uint32_t ldb8(const uint8_t *p) { return __ldg(p); }
__device__ __forceinline__ uint32_t ldb16(const uint8_t *p) { return ldb8(p) | (ldb8(p + 1) << 8); }

// Weight k of a row of GGUF blocks, exactly as the loader dequantises it.
template <int FMT> __device__ __forceinline__ float block_weight(const uint8_t *row, uint32_t k) {
  if constexpr (FMT == CUTB_Q8_0) {
    const uint8_t *b = row + (k >> 5) * 34;
    return (float)(int8_t)ldb8(b + 2 + (k & 31)) * h2f_bits(ldb16(b));
  } else if constexpr (FMT == CUTB_Q4_0) {
    const uint8_t *b = row + (k >> 5) * 18;
    const uint32_t e = k & 31, byte = ldb8(b + 2 + (e & 15));
    const int q = (int)((e < 16) ? (byte & 0xF) : (byte >> 4)) - 8;
    return (float)q * h2f_bits(ldb16(b));
  } else {
    const uint8_t *b = row + (k >> 8) * 144;
    const uint32_t e = k & 255, j = e >> 5, l = e & 31;
    const uint8_t *sc = b + 4;
    uint32_t s, m;
    if (j < 4) {
      s = ldb8(sc + j) & 63;
      m = ldb8(sc + j + 4) & 63;
    } else {
      s = (ldb8(sc + j + 4) & 0xF) | ((ldb8(sc + j - 4) >> 6) << 4);
      m = (ldb8(sc + j + 4) >> 4) | ((ldb8(sc + j) >> 6) << 4);
    }
    const uint32_t byte = ldb8(b + 16 + (j >> 1) * 32 + l);
    const uint32_t q = (j & 1) ? (byte >> 4) : (byte & 0xF);
    const float d1 = __fmul_rn(h2f_bits(ldb16(b)), (float)s);
    const float dm = __fmul_rn(h2f_bits(ldb16(b + 2)), (float)m);
    return __fsub_rn(__fmul_rn(d1, (float)q), dm);
  }
}

// One warp per weight row n; lanes stride over k; GEN_MT activation rows per pass.
template <int FMT, bool AF32>
__global__ void __launch_bounds__(256) qmatmul_blocks_generic_kernel(const GenParams p) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
  for (uint32_t n = warp; n < p.N; n += nwarps) {
    const uint8_t *row = p.W + (uint64_t)n * p.row_bytes;
    for (uint32_t m0 = 0; m0 < p.M; m0 += GEN_MT) {
      float acc[GEN_MT];
#pragma unroll
      for (int i = 0; i < GEN_MT; ++i) acc[i] = 0.f;
      for (uint32_t k = lane; k < p.K; k += 32) {
        const float w = block_weight<FMT>(row, k);
#pragma unroll
        for (int i = 0; i < GEN_MT; ++i)
          if (m0 + i < p.M) acc[i] = fmaf(load_a<AF32>(p.A, (uint64_t)(m0 + i) * p.lda + k), w, acc[i]);
      }
#pragma unroll
      for (int i = 0; i < GEN_MT; ++i) {
        float v = acc[i];
        for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && m0 + i < p.M) {
          const uint32_t m = m0 + i;
          const float dv = (p.fusion_type == CUTB_FUSION_BINARY) ? p.D[(uint64_t)m * p.ldd + n] : 0.f;
          p.C[(uint64_t)m * p.ldc + n] = apply_epilogue(v, p.fusion_type, p.fusion_op, dv);
        }
      }
    }
  }
}

// Reference runtime layout: thread (x) owns output column n, blockIdx.y walks
// groups of GEN_MT activation rows; consecutive threads read consecutive
// bytes of a k-row of the value plane.
template <bool Q4, bool AF32>
__global__ void __launch_bounds__(128) qmatmul_planes_kernel(const GenParams p) {
  const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t m0 = blockIdx.y * GEN_MT;
  if (n >= p.N) return;
  const uint32_t blocksK = (p.K + 31) >> 5;
  float acc[GEN_MT];
#pragma unroll
  for (int i = 0; i < GEN_MT; ++i) acc[i] = 0.f;
  for (uint32_t kb = 0; kb < blocksK; ++kb) {
    const float s = h2f_bits(__ldg(p.S + (uint64_t)kb * p.lds + n));
    const float mn = (Q4 && p.affine) ? h2f_bits(__ldg(p.S + (uint64_t)(kb + blocksK) * p.lds + n)) : 0.f;
    const uint32_t kend = min(p.K, kb * 32 + 32);
    for (uint32_t k = kb * 32; k < kend; ++k) {
      float w;
      if constexpr (Q4) {
        const uint32_t byte = ldb8(p.W + (uint64_t)k * p.ldb + (n >> 1));
        const int q = (int)((byte >> ((n & 1) * 4)) & 0xF) - 8;
        w = __fmul_rn((float)q, s);
        if (p.affine) w = __fadd_rn(w, mn);
      } else {
        w = (float)(int8_t)ldb8(p.W + (uint64_t)k * p.ldb + n) * s;
      }
#pragma unroll
      for (int i = 0; i < GEN_MT; ++i)
        if (m0 + i < p.M) acc[i] = fmaf(load_a<AF32>(p.A, (uint64_t)(m0 + i) * p.lda + k), w, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < GEN_MT; ++i)
    if (m0 + i < p.M) {
      const uint32_t m = m0 + i;
      const float dv = (p.fusion_type == CUTB_FUSION_BINARY) ? p.D[(uint64_t)m * p.ldd + n] : 0.f;
      p.C[(uint64_t)m * p.ldc + n] = apply_epilogue(acc[i], p.fusion_type, p.fusion_op, dv);
    }
}

}  // namespace

int qmatmul_generic_launch(const cutb_qmatmul_desc &d, cudaStream_t stream) {
  GenParams p;
  p.W = reinterpret_cast<const uint8_t *>(d.W);
  p.S = reinterpret_cast<const uint16_t *>(d.scales);
  p.A = d.A;
  p.C = d.C;
  p.D = d.D;
  p.row_bytes = row_bytes(d.format, d.K);
  p.M = d.M; p.K = d.K; p.N = d.N;
  p.lda = d.lda; p.ldb = d.ldb; p.lds = d.lds; p.ldc = d.ldc; p.ldd = d.ldd;
  p.fusion_type = d.fusion_type; p.fusion_op = d.fusion_op; p.affine = d.affine;
  const bool af32 = d.a_dtype == CUTB_F32;
  if (d.layout == CUTB_LAYOUT_KN_PLANES) {
    dim3 grid((d.N + 127) / 128, (d.M + GEN_MT - 1) / GEN_MT);
    if (d.format == CUTB_Q8_0) {
      if (af32) qmatmul_planes_kernel<false, true><<<grid, 128, 0, stream>>>(p);
      else qmatmul_planes_kernel<false, false><<<grid, 128, 0, stream>>>(p);
    } else {
      if (af32) qmatmul_planes_kernel<true, true><<<grid, 128, 0, stream>>>(p);
      else qmatmul_planes_kernel<true, false><<<grid, 128, 0, stream>>>(p);
    }
  } else {
    DeviceInfo di;
    if (int rc = get_device_info(&di)) return rc;
    const uint32_t want = (d.N + 7) / 8;  // 8 warps per CTA
    const uint32_t cap = (uint32_t)di.sm_count * 8;
    const uint32_t grid = want < cap ? want : cap;
#define CUTB_GEN(F)                                                                                   \
  if (af32) qmatmul_blocks_generic_kernel<F, true><<<grid, 256, 0, stream>>>(p);                      \
  else qmatmul_blocks_generic_kernel<F, false><<<grid, 256, 0, stream>>>(p)
    if (d.format == CUTB_Q8_0) { CUTB_GEN(CUTB_Q8_0); }
    else if (d.format == CUTB_Q4_0) { CUTB_GEN(CUTB_Q4_0); }
    else { CUTB_GEN(CUTB_Q4_K); }
#undef CUTB_GEN
  }
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace cutb
