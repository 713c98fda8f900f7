// Decode mat-vec over the reference's run-time weight layout ([K, N] value plane + fp16 scale plane).
//
// C[m, n] = sum_k A[m, k] * w(k, n) for one to four activation rows, where
//   Q8: w = int8 B[k, n] * f16 S[k / 32, n]                       (MatMulQ8Common.cuh:127-200)
//   Q4: w = (nibble(B[k, n / 2], n & 1) - 8) * f16 S[k / 32, n]   (MatMulQ4Common.cuh:126-153)
//       + f16 S[K / 32 + k / 32, n] when affine (the runner's Q4_K re-encode).
// This is the layout the reference's loader and runner hand to MatMulOpNode
// (operators/impl/matmul/MatMulOp.cpp:309-329) and the one its own decode kernels walk
// (MatMulQ8GemvKPar8.cu:11-92, MatMulQ4GemvKPar8.cu:8-98: eight K slices per output column).  A caller
// that keeps that loader gets this kernel; the block-layout mat-vec needs no repack at all and is faster.
//
// HBM-bound byte work, laid out for coalescing: consecutive columns are consecutive bytes, so a thread
// owns four (Q8) or eight (Q4) neighbouring columns -- one 32-bit load per k row, a warp reads one full
// 128-byte line per row -- and the K axis is what gets split: over the eight warps of a block (32-row
// scale blocks dealt round-robin, partial sums met in shared memory in a fixed order) and, when the matrix
// has too few column groups to fill the GPU, over blockIdx.y (partial sums to the workspace, added in a
// fixed order by a second small kernel).  Every thread keeps 16 to 32 row loads in flight (the loads of the next
// sixteen rows are issued before the current sixteen are consumed).
#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

constexpr int GP_WARPS = 8;

struct GpParams {
  const uint8_t *B;
  const uint16_t *S;
  const void *A;
  float *C;
  const float *D;
  float *partial;  // [ksplit][M][N] when ksplit > 1
  uint32_t M, K, N, lda, ldb, lds, ldc, ldd;
  uint32_t kblocks_per_split;
  uint32_t ksplit;
  int fusion_type, fusion_op, affine;
};

template <bool AF32> __device__ __forceinline__ float gp_load_a(const void *A, uint64_t i) {
  if constexpr (AF32) return __ldg(reinterpret_cast<const float *>(A) + i);
  return __half2float(__ldg(reinterpret_cast<const __half *>(A) + i));
}

template <bool Q4, bool AF32, int MR>
__global__ void __launch_bounds__(GP_WARPS * 32, (Q4 && MR == 4) ? 1 : 2) qgemv_planes_kernel(const GpParams p) {
  constexpr int CPT = Q4 ? 8 : 4;  // columns per thread = one 32-bit word of a k row
  __shared__ float red[GP_WARPS][MR][32 * CPT];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = (blockIdx.x * 32 + lane) * CPT;
  const bool col_ok = n0 < p.N;  // (row strides are padded to 4 bytes / 4 scales: a word never leaves its row)
  const uint32_t blocksK = (p.K + 31) >> 5;
  const uint32_t kb0 = blockIdx.y * p.kblocks_per_split;
  const uint32_t kb1 = min(blocksK, kb0 + p.kblocks_per_split);

  float acc[MR][CPT];
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int c = 0; c < CPT; ++c) acc[m][c] = 0.f;

  // Per 32-row block: this lane's activation of every activation row (broadcast row by row in the loop) and the
  // block's scales (and affine mins) of the thread's columns.
  struct Meta {
    float a_lane[MR], s[CPT], mn[CPT];
  };
  auto load_meta = [&](Meta &mt, uint32_t kb) {
    const uint32_t k_base = kb * 32, rows = min(32u, p.K - k_base);
#pragma unroll
    for (int m = 0; m < MR; ++m)
      mt.a_lane[m] = (lane < rows && (uint32_t)m < p.M) ? gp_load_a<AF32>(p.A, (uint64_t)m * p.lda + k_base + lane) : 0.f;
#pragma unroll
    for (int c = 0; c < CPT; ++c) mt.s[c] = mt.mn[c] = 0.f;
    if (col_ok) {
#pragma unroll
      for (int h = 0; h < CPT / 4; ++h) {
        if (n0 + 4 * h < p.lds) {
          const uint2 sv = __ldg(reinterpret_cast<const uint2 *>(p.S + (uint64_t)kb * p.lds + n0 + 4 * h));
          mt.s[4 * h + 0] = h2f_bits(sv.x & 0xFFFFu), mt.s[4 * h + 1] = h2f_bits(sv.x >> 16);
          mt.s[4 * h + 2] = h2f_bits(sv.y & 0xFFFFu), mt.s[4 * h + 3] = h2f_bits(sv.y >> 16);
          if (Q4 && p.affine) {
            const uint2 mv = __ldg(reinterpret_cast<const uint2 *>(p.S + (uint64_t)(kb + blocksK) * p.lds + n0 + 4 * h));
            mt.mn[4 * h + 0] = h2f_bits(mv.x & 0xFFFFu), mt.mn[4 * h + 1] = h2f_bits(mv.x >> 16);
            mt.mn[4 * h + 2] = h2f_bits(mv.y & 0xFFFFu), mt.mn[4 * h + 3] = h2f_bits(mv.y >> 16);
          }
        }
      }
    }
  };
  // sixteen k rows of the thread's word column (rows past K read as zero quants; their activations are zero too)
  auto load_half = [&](uint32_t (&w)[16], uint32_t kb, uint32_t half) {
    const uint32_t k_base = kb * 32 + half * 16;
    const uint32_t rows = k_base < p.K ? min(16u, p.K - k_base) : 0u;
    const uint8_t *bp = p.B + (uint64_t)k_base * p.ldb + (Q4 ? n0 / 2 : n0);
#pragma unroll
    for (uint32_t r = 0; r < 16; ++r)
      w[r] = (col_ok && r < rows) ? __ldg(reinterpret_cast<const uint32_t *>(bp + (size_t)r * p.ldb)) : 0u;
  };
  // sum_k a_k q_k in fp32 (quants widened exactly: the byte or nibble is dropped into the mantissa of 2^23 and
  // 2^23 (+ 128) is subtracted), scaled once per block; the Q4 offset -8 and the affine min ride on sum_k a_k
  float inner[MR][CPT], asum[MR];
  auto compute_half = [&](const uint32_t (&w)[16], const Meta &mt, uint32_t half) {
#pragma unroll
    for (uint32_t r = 0; r < 16; ++r) {
      float a[MR];
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        a[m] = __shfl_sync(0xffffffffu, mt.a_lane[m], half * 16 + r);
        if constexpr (Q4) asum[m] += a[m];
      }
      const uint32_t x = Q4 ? w[r] : (w[r] ^ 0x80808080u);  // int8 -> biased unsigned byte
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        float qf;
        if constexpr (Q4) qf = __uint_as_float(((x >> (4 * c)) & 0xFu) | 0x4B000000u) - 8388608.f;
        else qf = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540u | (uint32_t)c)) - 8388736.f;
#pragma unroll
        for (int m = 0; m < MR; ++m) inner[m][c] = fmaf(a[m], qf, inner[m][c]);
      }
    }
  };

  // Software pipeline over the warp's blocks: the second half's rows are requested before the first half is
  // consumed, and the next block's first half (with its scales and activations) before the second half is.
  uint32_t w0[16], w1[16];
  Meta cur, nxt;
  uint32_t kb = kb0 + warp;
  if (kb < kb1) {
    load_meta(cur, kb);
    load_half(w0, kb, 0);
  }
#pragma unroll 1
  for (; kb < kb1; kb += GP_WARPS) {
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      asum[m] = 0.f;
#pragma unroll
      for (int c = 0; c < CPT; ++c) inner[m][c] = 0.f;
    }
    load_half(w1, kb, 1);
    compute_half(w0, cur, 0);
    const uint32_t nkb = kb + GP_WARPS;
    if (nkb < kb1) {
      load_meta(nxt, nkb);
      load_half(w0, nkb, 0);
    }
    compute_half(w1, cur, 1);
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        if constexpr (Q4) {
          acc[m][c] = fmaf(cur.s[c], fmaf(-8.f, asum[m], inner[m][c]), acc[m][c]);
          if (p.affine) acc[m][c] = fmaf(cur.mn[c], asum[m], acc[m][c]);
        } else {
          acc[m][c] = fmaf(cur.s[c], inner[m][c], acc[m][c]);
        }
      }
    cur = nxt;
  }

  // the eight K slices of the block meet in a fixed order
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int c = 0; c < CPT; ++c) red[warp][m][c * 32 + lane] = acc[m][c];
  __syncthreads();
  for (uint32_t o = threadIdx.x; o < MR * 32 * CPT; o += GP_WARPS * 32) {
    const uint32_t m = o / (32 * CPT), j = o % (32 * CPT);  // j = column inside the block's group, in output order
    const uint32_t l = j / CPT, c = j % CPT;
    const uint32_t n = blockIdx.x * 32 * CPT + j;
    if (m >= p.M || n >= p.N) continue;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < GP_WARPS; ++w) sum += red[w][m][c * 32 + l];
    if (p.ksplit > 1) {
      p.partial[((size_t)blockIdx.y * p.M + m) * p.N + n] = sum;
    } else {
      const float dv = (p.fusion_type == CUTB_FUSION_BINARY) ? p.D[(size_t)m * p.ldd + n] : 0.f;
      p.C[(size_t)m * p.ldc + n] = apply_epilogue(sum, p.fusion_type, p.fusion_op, dv);
    }
  }
}

__global__ void gp_reduce_kernel(const float *__restrict__ partial, float *__restrict__ C, const float *__restrict__ D, uint32_t M,
                                 uint32_t N, uint32_t ldc, uint32_t ldd, uint32_t ksplit, int ftype, int fop) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  const uint32_t m = i / N, n = i % N;
  float sum = 0.f;
  for (uint32_t s = 0; s < ksplit; ++s) sum += partial[((size_t)s * M + m) * N + n];
  const float dv = (ftype == CUTB_FUSION_BINARY) ? D[(size_t)m * ldd + n] : 0.f;
  C[(size_t)m * ldc + n] = apply_epilogue(sum, ftype, fop, dv);
}

struct GpPlan {
  uint32_t grid_x, ksplit, kblocks_per_split;
};

GpPlan gp_plan(const cutb_qmatmul_desc &d, int sm_count) {
  const uint32_t cpt = d.format == CUTB_Q8_0 ? 4 : 8;
  GpPlan pl;
  pl.grid_x = (d.N + 32 * cpt - 1) / (32 * cpt);
  const uint32_t blocksK = (d.K + 31) / 32;
  // about sixteen resident warps per SM, and at least one 32-row block per warp
  const uint32_t want_ctas = (uint32_t)sm_count * 2;
  // (rounded down: two blocks fit an SM, and a handful of blocks beyond 2 x SMs would run as a wave of their own)
  uint32_t ks = pl.grid_x >= want_ctas ? 1 : want_ctas / pl.grid_x;
  const uint32_t max_ks = (blocksK + GP_WARPS - 1) / GP_WARPS;
  if (ks > max_ks) ks = max_ks;
  if (ks < 1) ks = 1;
  pl.kblocks_per_split = (blocksK + ks - 1) / ks;
  pl.ksplit = (blocksK + pl.kblocks_per_split - 1) / pl.kblocks_per_split;
  return pl;
}

}  // namespace

bool qgemv_planes_supported(const cutb_qmatmul_desc &d) {
  if (d.layout != CUTB_LAYOUT_KN_PLANES) return false;
  if (d.format != CUTB_Q8_0 && d.format != CUTB_Q4_0) return false;
  if (d.M == 0 || d.M > 4 || d.K == 0 || d.N == 0) return false;
  // one 32-bit word per k row and four scales per load: the reference's pad-to-4 strides and allocations give this
  if (reinterpret_cast<uintptr_t>(d.W) % 4 != 0 || d.ldb % 4 != 0) return false;
  if (reinterpret_cast<uintptr_t>(d.scales) % 8 != 0 || d.lds % 4 != 0) return false;
  const uint64_t row = d.format == CUTB_Q8_0 ? d.N : (d.N + 1) / 2;
  if (d.ldb < ((row + 3) & ~3ull) || d.lds < ((d.N + 3) & ~3u)) return false;
  return true;
}

uint64_t qgemv_planes_workspace(const cutb_qmatmul_desc &d) {
  if (!qgemv_planes_supported(d)) return 0;
  DeviceInfo di;
  if (get_device_info(&di) != CUTB_OK) di.sm_count = 148;
  const GpPlan pl = gp_plan(d, di.sm_count);
  return pl.ksplit > 1 ? (uint64_t)pl.ksplit * d.M * d.N * sizeof(float) : 0;
}

int qgemv_planes_launch(const cutb_qmatmul_desc &d, cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  const GpPlan pl = gp_plan(d, di.sm_count);
  GpParams p;
  p.B = reinterpret_cast<const uint8_t *>(d.W);
  p.S = reinterpret_cast<const uint16_t *>(d.scales);
  p.A = d.A;
  p.C = d.C;
  p.D = d.D;
  p.partial = nullptr;
  p.M = d.M; p.K = d.K; p.N = d.N;
  p.lda = d.lda; p.ldb = d.ldb; p.lds = d.lds; p.ldc = d.ldc; p.ldd = d.ldd;
  p.kblocks_per_split = pl.kblocks_per_split;
  p.ksplit = pl.ksplit;
  p.fusion_type = d.fusion_type; p.fusion_op = d.fusion_op; p.affine = d.affine;
  if (pl.ksplit > 1) {
    const uint64_t need = (uint64_t)pl.ksplit * d.M * d.N * sizeof(float);
    if (!d.workspace || d.workspace_bytes < need) {
      set_last_error("qgemv (planes): this shape splits K %u ways and needs %llu workspace bytes, got %llu", pl.ksplit,
                     (unsigned long long)need, (unsigned long long)d.workspace_bytes);
      return CUTB_ERR_WORKSPACE;
    }
    p.partial = reinterpret_cast<float *>(d.workspace);
  }
  const dim3 grid(pl.grid_x, pl.ksplit), block(GP_WARPS * 32);
  const bool q4 = d.format != CUTB_Q8_0, af32 = d.a_dtype == CUTB_F32;
  const int mr = d.M == 1 ? 1 : (d.M == 2 ? 2 : 4);
#define CUTB_GP(Q4, AF32, MR) qgemv_planes_kernel<Q4, AF32, MR><<<grid, block, 0, stream>>>(p)
#define CUTB_GP_M(Q4, AF32)            \
  if (mr == 1) CUTB_GP(Q4, AF32, 1);   \
  else if (mr == 2) CUTB_GP(Q4, AF32, 2); \
  else CUTB_GP(Q4, AF32, 4)
  if (q4) {
    if (af32) { CUTB_GP_M(true, true); } else { CUTB_GP_M(true, false); }
  } else {
    if (af32) { CUTB_GP_M(false, true); } else { CUTB_GP_M(false, false); }
  }
#undef CUTB_GP_M
#undef CUTB_GP
  CUTB_CUDA_TRY(cudaGetLastError());
  if (pl.ksplit > 1) {
    gp_reduce_kernel<<<(d.M * d.N + 255) / 256, 256, 0, stream>>>(p.partial, d.C, d.D, d.M, d.N, d.ldc, d.ldd, pl.ksplit, d.fusion_type,
                                                                  d.fusion_op);
    CUTB_CUDA_TRY(cudaGetLastError());
  }
  return CUTB_OK;
}

}  // namespace cutb
