// Decode mat-vec (M <= 32 activation rows) over native GGUF blocks for sm_100a.
//
// C[m, n] = sum_k A[m, k] * dequant(W)[n, k], W = N rows of Q8_0 / Q4_0 / Q4_K
// blocks.  Replaces the reference's M = 1 variants MatMulQ4GemvKPar8 /
// MatMulQ8GemvKPar8 (operators/impl/matmul/MatMulQ4GemvKPar8.cu:8-98,
// MatMulQ8GemvKPar8.cu:11-92) on the block layout its loader reads
// (interface/loader/gguf/gguf_reader.cpp:541-572, 678-724, 826-850).
//
// Design (HBM-bound: every weight byte is read exactly once):
//  * One persistent CTA per SM owns a contiguous range of weight rows, walked
//    in tiles of 16 rows.  The K axis of a tile is split over the CTA's 8 warps.
//  * Each warp runs its own 4-deep ring of shared-memory stages filled by bulk
//    async copies (cp.async.bulk, the TMA engine's untiled form; one copy per
//    row and stage, completion counted on an mbarrier).  A stage holds 16 rows
//    x 256 or 512 weights of raw block bytes, rows padded so that the fragment
//    reads below are bank-conflict free.  All of a CTA's first copies are in
//    flight before it touches the activations.
//  * Integer quants are widened to exact fp16 integers in registers (magic
//    number 0x6400 | q), and one m16n8k16 MMA per 16 weights-per-row contracts
//    them with the fp16 activations, fp32 accumulate.  Products of an fp16
//    integer and an fp16 activation are exact in fp32, so the only rounding is
//    the fp32 accumulation, as in the reference's fmaf loop.  The per-block
//    fp16 scale (and the Q4_K 6-bit sub-scales / mins, unpacked in registers)
//    is applied in fp32 to each 32-weight partial sum.
//  * The 8 activation "columns" of the MMA carry up to 8 batch rows.  fp32
//    activations are split into fp16 hi + lo parts (two columns per row) after
//    a power-of-two rescale, which keeps ~22 bits of each activation.
//  * Partial sums of the 8 warps meet in shared memory in a fixed order
//    (deterministic), then the fused epilogue runs and C is written.  With
//    ksplit > 1 (long K or few rows) raw partial sums go to a workspace and a
//    second small kernel adds them in a fixed order.
//
// Every wait on an mbarrier is bounded; on expiry the kernel stores
// CUTB_ERR_TIMEOUT in the caller's status word and leaves without spinning.
#include "common.cuh"
#include "kernels.h"

namespace cutb {

namespace {

constexpr int GV_WARPS = 8;
constexpr int GV_THREADS = GV_WARPS * 32;
constexpr int GV_STAGES = 4;
constexpr int GV_ROWS = 16;

// Granules (256 weights) per stage and padded shared-memory row stride.
template <int FMT> struct GvFmt;
template <> struct GvFmt<CUTB_Q8_0> { static constexpr int SG = 1; static constexpr int RS = 272; };
template <> struct GvFmt<CUTB_Q4_0> { static constexpr int SG = 2; static constexpr int RS = 304; };
template <> struct GvFmt<CUTB_Q4_K> { static constexpr int SG = 2; static constexpr int RS = 288; };

struct GvParams {
  const uint8_t *W;
  uint64_t row_bytes;
  const void *A;
  uint32_t lda;
  float *C;
  uint32_t ldc;
  const float *D;
  uint32_t ldd;
  float *partial;  // [ksplit][M][N] when ksplit > 1
  uint32_t M, K, N;
  uint32_t gran_per_split;
  uint32_t ksplit;
  int fusion_type, fusion_op;
  int vec_ok;  // activation rows allow 8/16-byte vector loads
  int *status;
};

__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Two 4-bit quants (bits 0-3 and 16-19 of x) -> half2 of (q - bias).
__device__ __forceinline__ uint32_t nib_lo(uint32_t x, float bias) {
  uint32_t v = (x & 0x000F000Fu) | 0x64006400u;  // 1024 + q
  return h2_as_u32(__hsub2(u32_as_h2(v), __float2half2_rn(1024.0f + bias)));
}
// Two 4-bit quants (bits 4-7 and 20-23 of x) -> half2 of (q - bias).
__device__ __forceinline__ uint32_t nib_hi(uint32_t x, float bias) {
  uint32_t v = (x & 0x00F000F0u) | 0x64006400u;  // 1024 + 16 q
  return h2_as_u32(__hfma2(u32_as_h2(v), __float2half2_rn(0.0625f), __float2half2_rn(-64.0f - bias)));
}
// Bytes sel0/sel1 of u (already biased by +128) -> half2 of the signed int8 values.
template <uint32_t SEL> __device__ __forceinline__ uint32_t i8_pair(uint32_t u) {
  uint32_t v = __byte_perm(u, 0x64646464u, SEL);  // 1024 + (q + 128)
  return h2_as_u32(__hsub2(u32_as_h2(v), __float2half2_rn(1152.0f)));
}

// One stage of one warp: 16 rows x (ngr granules) of raw blocks at `st`
// (shared address), activations for the first block of the stage at `actb`
// (shared address, block stride `act_stride` bytes).
template <int FMT, int NT>
__device__ __forceinline__ void compute_stage(uint32_t st, uint32_t ngr, uint32_t actb, uint32_t act_stride,
                                              const uint32_t (&aoff)[NT], uint32_t ssb, uint32_t g, uint32_t t,
                                              float (&tot)[NT][4]) {
  constexpr int RS = GvFmt<FMT>::RS;
  const uint32_t rowA = st + g * RS, rowB = rowA + 8 * RS;
  if constexpr (FMT == CUTB_Q4_0) {
    const uint32_t nb = ngr * 8;
#pragma unroll 4
    for (uint32_t b = 0; b < nb; ++b) {
      const uint32_t pa = rowA + b * 18, pb = rowB + b * 18;
      const float dA = h2f_bits(lds_u16(pa)), dB = h2f_bits(lds_u16(pb));
      const uint32_t xa = lds_u16(pa + 2 + 4 * t) | (lds_u16(pa + 4 + 4 * t) << 16);
      const uint32_t xb = lds_u16(pb + 2 + 4 * t) | (lds_u16(pb + 4 + 4 * t) << 16);
      const uint32_t a_l0 = nib_lo(xa, 8.f), a_l1 = nib_lo(xa >> 8, 8.f), a_h0 = nib_hi(xa, 8.f), a_h1 = nib_hi(xa >> 8, 8.f);
      const uint32_t b_l0 = nib_lo(xb, 8.f), b_l1 = nib_lo(xb >> 8, 8.f), b_h0 = nib_hi(xb, 8.f), b_h1 = nib_hi(xb >> 8, 8.f);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 x = lds_u128(actb + b * act_stride + aoff[nt]);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        mma16816(acc, a_l0, b_l0, a_l1, b_l1, x.x, x.y);
        mma16816(acc, a_h0, b_h0, a_h1, b_h1, x.z, x.w);
        tot[nt][0] = fmaf(dA, acc[0], tot[nt][0]);
        tot[nt][1] = fmaf(dA, acc[1], tot[nt][1]);
        tot[nt][2] = fmaf(dB, acc[2], tot[nt][2]);
        tot[nt][3] = fmaf(dB, acc[3], tot[nt][3]);
      }
    }
  } else if constexpr (FMT == CUTB_Q8_0) {
    const uint32_t nb = ngr * 8;
#pragma unroll 4
    for (uint32_t b = 0; b < nb; ++b) {
      const uint32_t pa = rowA + b * 34, pb = rowB + b * 34;
      const float dA = h2f_bits(lds_u16(pa)), dB = h2f_bits(lds_u16(pb));
      // bytes 4t..4t+3 and 16+4t..16+4t+3 of the 32 quants
      const uint32_t a0w = (lds_u16(pa + 2 + 4 * t) | (lds_u16(pa + 4 + 4 * t) << 16)) ^ 0x80808080u;
      const uint32_t a1w = (lds_u16(pa + 18 + 4 * t) | (lds_u16(pa + 20 + 4 * t) << 16)) ^ 0x80808080u;
      const uint32_t b0w = (lds_u16(pb + 2 + 4 * t) | (lds_u16(pb + 4 + 4 * t) << 16)) ^ 0x80808080u;
      const uint32_t b1w = (lds_u16(pb + 18 + 4 * t) | (lds_u16(pb + 20 + 4 * t) << 16)) ^ 0x80808080u;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 x = lds_u128(actb + b * act_stride + aoff[nt]);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        mma16816(acc, i8_pair<0x4140>(a0w), i8_pair<0x4140>(b0w), i8_pair<0x4342>(a0w), i8_pair<0x4342>(b0w), x.x, x.y);
        mma16816(acc, i8_pair<0x4140>(a1w), i8_pair<0x4140>(b1w), i8_pair<0x4342>(a1w), i8_pair<0x4342>(b1w), x.z, x.w);
        tot[nt][0] = fmaf(dA, acc[0], tot[nt][0]);
        tot[nt][1] = fmaf(dA, acc[1], tot[nt][1]);
        tot[nt][2] = fmaf(dB, acc[2], tot[nt][2]);
        tot[nt][3] = fmaf(dB, acc[3], tot[nt][3]);
      }
    }
  } else {  // Q4_K: ngr super-blocks of 144 bytes per row
    for (uint32_t s = 0; s < ngr; ++s) {
      const uint32_t pa = rowA + s * 144, pb = rowB + s * 144;
      const uint4 hA = lds_u128(pa), hB = lds_u128(pb);
      const float dA = h2f_bits(hA.x & 0xFFFFu), mA = h2f_bits(hA.x >> 16);
      const float dB = h2f_bits(hB.x & 0xFFFFu), mB = h2f_bits(hB.x >> 16);
      // 6-bit (scale, min) pairs, four per 32-bit word
      // (gguf_reader.cpp:668-676 unpacked four sub-blocks at a time)
      const uint32_t scA[2] = {hA.y & 0x3F3F3F3Fu, (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u)};
      const uint32_t mnA[2] = {hA.z & 0x3F3F3F3Fu, ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u)};
      const uint32_t scB[2] = {hB.y & 0x3F3F3F3Fu, (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u)};
      const uint32_t mnB[2] = {hB.z & 0x3F3F3F3Fu, ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u)};
      // d * (2^23 + sc) - d * 2^23 == d * sc exactly (<= 17 significant bits)
      const float ndA = -dA * 8388608.f, nmA = -mA * 8388608.f, ndB = -dB * 8388608.f, nmB = -mB * 8388608.f;
#pragma unroll
      for (int gq = 0; gq < 4; ++gq) {
        const uint2 qa = lds_u64(pa + 16 + 32 * gq + 8 * t), qb = lds_u64(pb + 16 + 32 * gq + 8 * t);
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
          const int j = 2 * gq + hi;  // sub-block 0..7
          const uint32_t sel = 0x7540u | (uint32_t)(j & 3);
          const float scfA = __uint_as_float(__byte_perm(scA[j >> 2], 0x4B000000u, sel));
          const float mnfA = __uint_as_float(__byte_perm(mnA[j >> 2], 0x4B000000u, sel));
          const float scfB = __uint_as_float(__byte_perm(scB[j >> 2], 0x4B000000u, sel));
          const float mnfB = __uint_as_float(__byte_perm(mnB[j >> 2], 0x4B000000u, sel));
          const float dsA = fmaf(dA, scfA, ndA), dmA = fmaf(mA, mnfA, nmA);
          const float dsB = fmaf(dB, scfB, ndB), dmB = fmaf(mB, mnfB, nmB);
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
          if (hi == 0) {
            a0 = nib_lo(qa.x, 0.f); a1 = nib_lo(qa.x >> 8, 0.f); a2 = nib_lo(qa.y, 0.f); a3 = nib_lo(qa.y >> 8, 0.f);
            b0 = nib_lo(qb.x, 0.f); b1 = nib_lo(qb.x >> 8, 0.f); b2 = nib_lo(qb.y, 0.f); b3 = nib_lo(qb.y >> 8, 0.f);
          } else {
            a0 = nib_hi(qa.x, 0.f); a1 = nib_hi(qa.x >> 8, 0.f); a2 = nib_hi(qa.y, 0.f); a3 = nib_hi(qa.y >> 8, 0.f);
            b0 = nib_hi(qb.x, 0.f); b1 = nib_hi(qb.x >> 8, 0.f); b2 = nib_hi(qb.y, 0.f); b3 = nib_hi(qb.y >> 8, 0.f);
          }
          const uint32_t kb = s * 8 + j;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 x = lds_u128(actb + kb * act_stride + aoff[nt]);
            const uint2 sv = lds_u64(ssb + ((kb * NT + nt) * 8 + 2 * t) * 4);
            const float s0 = __uint_as_float(sv.x), s1 = __uint_as_float(sv.y);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            mma16816(acc, a0, b0, a1, b1, x.x, x.y);
            mma16816(acc, a2, b2, a3, b3, x.z, x.w);
            tot[nt][0] = fmaf(dsA, acc[0], tot[nt][0]);
            tot[nt][1] = fmaf(dsA, acc[1], tot[nt][1]);
            tot[nt][2] = fmaf(dsB, acc[2], tot[nt][2]);
            tot[nt][3] = fmaf(dsB, acc[3], tot[nt][3]);
            tot[nt][0] = fmaf(-dmA, s0, tot[nt][0]);
            tot[nt][1] = fmaf(-dmA, s1, tot[nt][1]);
            tot[nt][2] = fmaf(-dmB, s0, tot[nt][2]);
            tot[nt][3] = fmaf(-dmB, s1, tot[nt][3]);
          }
        }
      }
    }
  }
}

// Loads 4 consecutive activations as floats.
template <bool AF32>
__device__ __forceinline__ void load4(const void *A, uint64_t idx, bool vec, float (&v)[4]) {
  if constexpr (AF32) {
    const float *p = reinterpret_cast<const float *>(A) + idx;
    if (vec) {
      const float4 f = __ldg(reinterpret_cast<const float4 *>(p));
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      v[0] = __ldg(p); v[1] = __ldg(p + 1); v[2] = __ldg(p + 2); v[3] = __ldg(p + 3);
    }
  } else {
    const __half *p = reinterpret_cast<const __half *>(A) + idx;
    if (vec) {
      const uint2 u = __ldg(reinterpret_cast<const uint2 *>(p));
      const float2 f0 = __half22float2(u32_as_h2(u.x)), f1 = __half22float2(u32_as_h2(u.y));
      v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
    } else {
      v[0] = __half2float(p[0]); v[1] = __half2float(p[1]); v[2] = __half2float(p[2]); v[3] = __half2float(p[3]);
    }
  }
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) { return h2_as_u32(__floats2half2_rn(a, b)); }

template <int FMT, bool AF32, int NT>
__global__ void __launch_bounds__(GV_THREADS, 1) qgemv_blocks_kernel(const GvParams p) {
  using F = GvFmt<FMT>;
  constexpr int SG = F::SG, RS = F::RS;
  constexpr uint32_t GB = granule_bytes(FMT);
  constexpr uint32_t STAGE_BYTES = GV_ROWS * RS;
  constexpr uint32_t NC8 = NT * 8;
  extern __shared__ __align__(128) uint8_t smem[];

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const uint32_t ncols = AF32 ? 2 * p.M : p.M;
  const uint32_t ncp = (ncols < NC8) ? ncols + 1 : ncols;  // one extra all-zero column for idle MMA lanes
  const uint32_t nblk_alloc = p.gran_per_split * 8;

  uint8_t *ring = smem;
  uint8_t *act = ring + GV_WARPS * GV_STAGES * STAGE_BYTES;
  float *ssum = reinterpret_cast<float *>(act + (size_t)nblk_alloc * ncp * 64);
  float *red = ssum + (FMT == CUTB_Q4_K ? nblk_alloc * NC8 : 0);
  float *scl = red + GV_WARPS * GV_ROWS * NC8;  // [0,16): 1/scale per activation row, [16,32): scale
  uint64_t *bars = reinterpret_cast<uint64_t *>(scl + 32);

  // rows of this CTA, granules (256 weights) of this K split and of this warp
  const uint32_t r0 = (uint32_t)((uint64_t)blockIdx.x * p.N / gridDim.x);
  const uint32_t r1 = (uint32_t)((uint64_t)(blockIdx.x + 1) * p.N / gridDim.x);
  const uint32_t G = p.K >> 8;
  const uint32_t gs0 = blockIdx.y * p.gran_per_split;
  const uint32_t gs1 = min(G, gs0 + p.gran_per_split);
  const uint32_t ng = gs1 - gs0;
  const uint32_t wg0 = gs0 + ng * warp / GV_WARPS, wg1 = gs0 + ng * (warp + 1) / GV_WARPS;
  const uint32_t spt = (wg1 - wg0 + SG - 1) / SG;  // stages per row tile for this warp
  const uint32_t ntiles = (r1 - r0 + GV_ROWS - 1) / GV_ROWS;
  const uint32_t total_stages = ntiles * spt;

  const uint32_t ring_w = smem_u32(ring) + warp * GV_STAGES * STAGE_BYTES;
  const uint32_t bar_w = smem_u32(bars) + warp * GV_STAGES * 8;

  if (lane == 0) {
    for (int s = 0; s < GV_STAGES; ++s) mbar_init(bar_w + s * 8, 1);
    fence_mbar_init();
  }
  __syncwarp();

  auto issue = [&](uint32_t j) {
    const uint32_t tile = j / spt, s = j - tile * spt, slot = j % GV_STAGES;
    const uint32_t gq = wg0 + s * SG;
    const uint32_t bytes = min((uint32_t)SG, wg1 - gq) * GB;
    const uint32_t row_base = r0 + tile * GV_ROWS;
    const uint32_t valid = min((uint32_t)GV_ROWS, r1 - row_base);
    const uint32_t bar = bar_w + slot * 8;
    if (lane == 0) mbar_arrive_expect_tx(bar, valid * bytes);
    __syncwarp();
    if (lane < valid)
      bulk_g2s(ring_w + slot * STAGE_BYTES + lane * RS, p.W + (uint64_t)(row_base + lane) * p.row_bytes + (uint64_t)gq * GB,
               bytes, bar);
  };

  // Put the first weight bytes in flight before anything else.
  const uint32_t pre = min((uint32_t)GV_STAGES, total_stages);
  for (uint32_t j = 0; j < pre; ++j) issue(j);

  // ---- stage the activations of this K split in MMA fragment order ----------
  const uint32_t k0 = gs0 * 256, nblk = ng * 8;
  if constexpr (AF32) {
    // per-row power-of-two rescale so that hi/lo fp16 parts neither overflow nor lose bits
    for (uint32_t m = 0; m < p.M; ++m) {
      const float *row = reinterpret_cast<const float *>(p.A) + (uint64_t)m * p.lda + k0;
      float mx = 0.f;
      for (uint32_t k = tid; k < nblk * 32; k += GV_THREADS) mx = fmaxf(mx, fabsf(__ldg(row + k)));
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red[warp] = mx;
      __syncthreads();
      if (tid == 0) {
        float a = red[0];
        for (int w = 1; w < GV_WARPS; ++w) a = fmaxf(a, red[w]);
        const int e = (int)((__float_as_uint(a) >> 23) & 0xFFu) - 127;
        int sh = 14 - e;
        if (a == 0.f || e == 128) sh = 0;
        sh = max(-113, min(126, sh));
        scl[16 + m] = __uint_as_float((uint32_t)(127 + sh) << 23);
        scl[m] = __uint_as_float((uint32_t)(127 - sh) << 23);
      }
      __syncthreads();
    }
  }
  {
    const uint32_t nrows = p.M;  // activation rows
    const uint32_t nchunks = nblk * nrows * 4;
    // uniform trip count: the shuffles below need every lane of a warp present
    for (uint32_t base = 0; base < nchunks; base += GV_THREADS) {
      const uint32_t id = base + tid;
      const uint32_t ct = id & 3, q = id >> 2;
      const uint32_t m = q % nrows, kb = q / nrows;
      const bool live = id < nchunks;
      float v0[4] = {0, 0, 0, 0}, v1[4] = {0, 0, 0, 0};
      if (live) {
        const uint64_t base = (uint64_t)m * p.lda + k0 + kb * 32;
        const uint32_t o0 = (FMT == CUTB_Q4_K) ? 8 * ct : 4 * ct;
        const uint32_t o1 = (FMT == CUTB_Q4_K) ? 8 * ct + 4 : 16 + 4 * ct;
        load4<AF32>(p.A, base + o0, p.vec_ok, v0);
        load4<AF32>(p.A, base + o1, p.vec_ok, v1);
      }
      // order inside a chunk: Q8_0 natural, 4-bit formats (0,2,1,3) to match the nibble pairs
      constexpr int P1 = (FMT == CUTB_Q8_0) ? 1 : 2, P2 = (FMT == CUTB_Q8_0) ? 2 : 1;
      uint4 c0, c1;
      float part;  // sum of the fp16 values this chunk contributes to its sub-block sum (Q4_K)
      float part_lo = 0.f;
      if constexpr (AF32) {
        const float sc = scl[16 + (live ? m : 0)];
        float h[8], l[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float x0 = v0[i] * sc, x1 = v1[i] * sc;
          h[i] = __half2float(__float2half_rn(x0));
          h[4 + i] = __half2float(__float2half_rn(x1));
          l[i] = __half2float(__float2half_rn(x0 - h[i]));
          l[4 + i] = __half2float(__float2half_rn(x1 - h[4 + i]));
        }
        c0 = make_uint4(pack_h2(h[0], h[P1]), pack_h2(h[P2], h[3]), pack_h2(h[4], h[4 + P1]), pack_h2(h[4 + P2], h[7]));
        c1 = make_uint4(pack_h2(l[0], l[P1]), pack_h2(l[P2], l[3]), pack_h2(l[4], l[4 + P1]), pack_h2(l[4 + P2], l[7]));
        part = ((h[0] + h[1]) + (h[2] + h[3])) + ((h[4] + h[5]) + (h[6] + h[7]));
        part_lo = ((l[0] + l[1]) + (l[2] + l[3])) + ((l[4] + l[5]) + (l[6] + l[7]));
      } else {
        c0 = make_uint4(pack_h2(v0[0], v0[P1]), pack_h2(v0[P2], v0[3]), pack_h2(v1[0], v1[P1]), pack_h2(v1[P2], v1[3]));
        c1 = c0;
        part = ((v0[0] + v0[1]) + (v0[2] + v0[3])) + ((v1[0] + v1[1]) + (v1[2] + v1[3]));
      }
      if constexpr (FMT == CUTB_Q4_K) {
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        part_lo += __shfl_xor_sync(0xffffffffu, part_lo, 1);
        part_lo += __shfl_xor_sync(0xffffffffu, part_lo, 2);
      }
      if (live) {
        const uint32_t col = AF32 ? 2 * m : m;
        *reinterpret_cast<uint4 *>(act + ((size_t)(kb * ncp + col) * 4 + ct) * 16) = c0;
        if constexpr (AF32) *reinterpret_cast<uint4 *>(act + ((size_t)(kb * ncp + col + 1) * 4 + ct) * 16) = c1;
        if constexpr (FMT == CUTB_Q4_K) {
          if (ct == 0) {
            ssum[kb * NC8 + col] = part;
            if constexpr (AF32) ssum[kb * NC8 + col + 1] = part_lo;
          }
        }
      }
    }
    // the all-zero column and the unused sub-block sums
    if (ncp > ncols)
      for (uint32_t id = tid; id < nblk * 4; id += GV_THREADS)
        *reinterpret_cast<uint4 *>(act + ((size_t)((id >> 2) * ncp + ncols) * 4 + (id & 3)) * 16) = make_uint4(0, 0, 0, 0);
    if constexpr (FMT == CUTB_Q4_K) {
      const uint32_t spare = NC8 - ncols;
      for (uint32_t id = tid; id < nblk * spare; id += GV_THREADS) ssum[(id / spare) * NC8 + ncols + id % spare] = 0.f;
    }
  }
  __syncthreads();

  // per-lane activation fragment offsets (idle lanes read the zero column)
  uint32_t aoff[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const uint32_t col = nt * 8 + g;
    aoff[nt] = ((col < ncols ? col : ncols) * 4 + t) * 16;
  }
  const uint32_t act_u = smem_u32(act), act_stride = ncp * 64, ss_u = smem_u32(ssum);

  bool dead = false;
  for (uint32_t tile = 0; tile < ntiles; ++tile) {
    float tot[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;

    for (uint32_t s = 0; s < spt; ++s) {
      const uint32_t j = tile * spt + s, slot = j % GV_STAGES, parity = (j / GV_STAGES) & 1u;
      if (!dead) {
        const bool ok = mbar_wait_bounded(bar_w + slot * 8, parity);
        if (!__all_sync(0xffffffffu, ok)) {
          dead = true;
          if (lane == 0 && p.status) atomicExch(p.status, (int)CUTB_ERR_TIMEOUT);
        }
      }
      if (!dead) {
        const uint32_t gq = wg0 + s * SG;
        const uint32_t ngr = min((uint32_t)SG, wg1 - gq);
        const uint32_t kb0 = (gq - gs0) * 8;  // first 32-weight block of the stage inside the split
        compute_stage<FMT, NT>(ring_w + slot * STAGE_BYTES, ngr, act_u + kb0 * act_stride, act_stride, aoff,
                               ss_u + kb0 * NC8 * 4, g, t, tot);
      }
      __syncwarp();
      if (!dead && j + GV_STAGES < total_stages) issue(j + GV_STAGES);
    }

    // meet the other warps' K slices in a fixed order
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float *r = red + ((size_t)warp * GV_ROWS) * NC8 + nt * 8 + 2 * t;
      *reinterpret_cast<float2 *>(r + g * NC8) = make_float2(tot[nt][0], tot[nt][1]);
      *reinterpret_cast<float2 *>(r + (g + 8) * NC8) = make_float2(tot[nt][2], tot[nt][3]);
    }
    __syncthreads();
    const uint32_t row_base = r0 + tile * GV_ROWS;
    for (uint32_t o = tid; o < GV_ROWS * p.M; o += GV_THREADS) {
      const uint32_t row = o % GV_ROWS, m = o / GV_ROWS, n = row_base + row;
      if (n < r1) {
        float sum = 0.f;
        if constexpr (AF32) {
#pragma unroll
          for (int w = 0; w < GV_WARPS; ++w) {
            const float2 hl = *reinterpret_cast<const float2 *>(red + ((size_t)w * GV_ROWS + row) * NC8 + 2 * m);
            sum += hl.x + hl.y;
          }
          sum *= scl[m];
        } else {
#pragma unroll
          for (int w = 0; w < GV_WARPS; ++w) sum += red[((size_t)w * GV_ROWS + row) * NC8 + m];
        }
        if (p.ksplit > 1) {
          p.partial[((size_t)blockIdx.y * p.M + m) * p.N + n] = sum;
        } else {
          const float dv = (p.fusion_type == CUTB_FUSION_BINARY) ? p.D[(size_t)m * p.ldd + n] : 0.f;
          p.C[(size_t)m * p.ldc + n] = apply_epilogue(sum, p.fusion_type, p.fusion_op, dv);
        }
      }
    }
    __syncthreads();
  }

  // A warp that gave up still owns copies in flight: give them a bounded
  // chance to land before the CTA's shared memory is released.
  if (dead) {
    for (int s = 0; s < GV_STAGES; ++s) {
      (void)mbar_wait_bounded(bar_w + s * 8, 0, 1u << 16);
      (void)mbar_wait_bounded(bar_w + s * 8, 1, 1u << 16);
    }
  }
}

// Fixed-order sum of the K-split partials followed by the fused epilogue.
__global__ void splitk_reduce_kernel(const float *__restrict__ partial, float *__restrict__ C, const float *__restrict__ D,
                                     uint32_t M, uint32_t N, uint32_t ldc, uint32_t ldd, uint32_t ksplit, int ftype, int fop) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  const uint32_t m = i / N, n = i % N;
  float sum = 0.f;
  for (uint32_t s = 0; s < ksplit; ++s) sum += partial[((size_t)s * M + m) * N + n];
  const float dv = (ftype == CUTB_FUSION_BINARY) ? D[(size_t)m * ldd + n] : 0.f;
  C[(size_t)m * ldc + n] = apply_epilogue(sum, ftype, fop, dv);
}

struct GvPlan {
  uint32_t nt, ncols, ncp, grid_x, ksplit, gran_per_split;
  size_t smem;
};

size_t gv_smem_bytes(int fmt, uint32_t nt, uint32_t ncp, uint32_t gran_per_split) {
  const uint32_t rs = fmt == CUTB_Q8_0 ? GvFmt<CUTB_Q8_0>::RS : (fmt == CUTB_Q4_0 ? GvFmt<CUTB_Q4_0>::RS : GvFmt<CUTB_Q4_K>::RS);
  const size_t nblk = (size_t)gran_per_split * 8;
  size_t b = (size_t)GV_WARPS * GV_STAGES * GV_ROWS * rs;
  b += nblk * ncp * 64;
  if (fmt == CUTB_Q4_K) b += nblk * nt * 8 * 4;
  b += (size_t)GV_WARPS * GV_ROWS * nt * 8 * 4;
  b += 32 * 4;
  b += GV_WARPS * GV_STAGES * 8;
  return b;
}

bool gv_plan(const cutb_qmatmul_desc &d, const DeviceInfo &di, GvPlan *pl) {
  const bool af32 = d.a_dtype == CUTB_F32;
  pl->ncols = af32 ? 2 * d.M : d.M;
  if (pl->ncols == 0 || pl->ncols > 32) return false;
  pl->nt = pl->ncols <= 8 ? 1 : (pl->ncols <= 16 ? 2 : 4);
  pl->ncp = pl->ncols < pl->nt * 8 ? pl->ncols + 1 : pl->ncols;
  const uint32_t G = d.K / 256;
  const uint32_t tiles = (d.N + GV_ROWS - 1) / GV_ROWS;
  pl->grid_x = tiles < (uint32_t)di.sm_count ? tiles : (uint32_t)di.sm_count;
  uint32_t want = 1;
  if (pl->grid_x * 2 <= (uint32_t)di.sm_count) want = (uint32_t)di.sm_count / pl->grid_x;
  if (want > G) want = G;
  const size_t limit = di.smem_optin;
  for (uint32_t ks = want; ks <= G; ++ks) {
    const uint32_t gps = (G + ks - 1) / ks;
    const size_t sm = gv_smem_bytes(d.format, pl->nt, pl->ncp, gps);
    if (sm <= limit) {
      pl->gran_per_split = gps;
      pl->ksplit = (G + gps - 1) / gps;
      pl->smem = sm;
      return true;
    }
  }
  return false;
}

template <int FMT, bool AF32, int NT>
int gv_launch_inst(const GvParams &p, const GvPlan &pl, cudaStream_t stream) {
  static int configured_device = -1;
  int dev = 0;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    DeviceInfo di;
    if (int rc = get_device_info(&di)) return rc;
    CUTB_CUDA_TRY(cudaFuncSetAttribute(qgemv_blocks_kernel<FMT, AF32, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)di.smem_optin));
    configured_device = dev;
  }
  qgemv_blocks_kernel<FMT, AF32, NT><<<dim3(pl.grid_x, pl.ksplit), GV_THREADS, pl.smem, stream>>>(p);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

template <int FMT, bool AF32>
int gv_launch_nt(const GvParams &p, const GvPlan &pl, cudaStream_t stream) {
  switch (pl.nt) {
    case 1: return gv_launch_inst<FMT, AF32, 1>(p, pl, stream);
    case 2: return gv_launch_inst<FMT, AF32, 2>(p, pl, stream);
    default: return gv_launch_inst<FMT, AF32, 4>(p, pl, stream);
  }
}

template <int FMT>
int gv_launch_a(const GvParams &p, const GvPlan &pl, bool af32, cudaStream_t stream) {
  return af32 ? gv_launch_nt<FMT, true>(p, pl, stream) : gv_launch_nt<FMT, false>(p, pl, stream);
}

}  // namespace

bool qgemv_blocks_supported(const cutb_qmatmul_desc &d) {
  if (d.layout != CUTB_LAYOUT_GGUF_BLOCKS) return false;
  if (d.K == 0 || d.K % 256 != 0 || d.N == 0 || d.M == 0) return false;
  const uint32_t ncols = d.a_dtype == CUTB_F32 ? 2 * d.M : d.M;
  if (ncols > 32) return false;
  if (reinterpret_cast<uintptr_t>(d.W) % 16 != 0) return false;
  return true;
}

uint64_t qgemv_blocks_workspace(const cutb_qmatmul_desc &d) {
  DeviceInfo di;
  if (get_device_info(&di) != CUTB_OK) {
    // no device: report the bound for a 148-SM part so callers can size ahead of time
    di.sm_count = 148;
    di.smem_optin = 232448;
  }
  GvPlan pl;
  if (!qgemv_blocks_supported(d) || !gv_plan(d, di, &pl)) return 0;
  return pl.ksplit > 1 ? (uint64_t)pl.ksplit * d.M * d.N * sizeof(float) : 0;
}

int qgemv_blocks_launch(const cutb_qmatmul_desc &d, cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  GvPlan pl;
  if (!gv_plan(d, di, &pl)) {
    set_last_error("qgemv: no shared-memory plan for M=%u K=%u N=%u", d.M, d.K, d.N);
    return CUTB_ERR_UNSUPPORTED;
  }
  const bool af32 = d.a_dtype == CUTB_F32;
  GvParams p;
  p.W = reinterpret_cast<const uint8_t *>(d.W);
  p.row_bytes = row_bytes(d.format, d.K);
  p.A = d.A;
  p.lda = d.lda;
  p.C = d.C;
  p.ldc = d.ldc;
  p.D = d.D;
  p.ldd = d.ldd;
  p.partial = nullptr;
  p.M = d.M;
  p.K = d.K;
  p.N = d.N;
  p.gran_per_split = pl.gran_per_split;
  p.ksplit = pl.ksplit;
  p.fusion_type = d.fusion_type;
  p.fusion_op = d.fusion_op;
  const uintptr_t a = reinterpret_cast<uintptr_t>(d.A);
  p.vec_ok = af32 ? (a % 16 == 0 && d.lda % 4 == 0) : (a % 8 == 0 && d.lda % 4 == 0);
  p.status = d.status;
  if (pl.ksplit > 1) {
    const uint64_t need = (uint64_t)pl.ksplit * d.M * d.N * sizeof(float);
    if (!d.workspace || d.workspace_bytes < need) {
      set_last_error("qgemv: split-K needs %llu workspace bytes, got %llu", (unsigned long long)need,
                     (unsigned long long)d.workspace_bytes);
      return CUTB_ERR_WORKSPACE;
    }
    p.partial = reinterpret_cast<float *>(d.workspace);
  }
  int rc;
  switch (d.format) {
    case CUTB_Q8_0: rc = gv_launch_a<CUTB_Q8_0>(p, pl, af32, stream); break;
    case CUTB_Q4_0: rc = gv_launch_a<CUTB_Q4_0>(p, pl, af32, stream); break;
    default: rc = gv_launch_a<CUTB_Q4_K>(p, pl, af32, stream); break;
  }
  if (rc != CUTB_OK) return rc;
  if (pl.ksplit > 1) {
    const uint32_t total = d.M * d.N;
    splitk_reduce_kernel<<<(total + 255) / 256, 256, 0, stream>>>(p.partial, d.C, d.D, d.M, d.N, d.ldc, d.ldd, pl.ksplit,
                                                                 d.fusion_type, d.fusion_op);
    CUTB_CUDA_TRY(cudaGetLastError());
  }
  return CUTB_OK;
}

}  // namespace cutb
