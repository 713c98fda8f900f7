// Decode mat-vec (a few activation rows) over native GGUF blocks for sm_100a.
//
// C[m, n] = sum_k A[m, k] * dequant(W)[n, k], W = N rows of Q8_0 / Q4_0 / Q4_K
// blocks.  Replaces the reference's M = 1 variants MatMulQ4GemvKPar8 /
// MatMulQ8GemvKPar8 (operators/impl/matmul/MatMulQ4GemvKPar8.cu:8-98,
// MatMulQ8GemvKPar8.cu:11-92) on the block layout its loader reads
// (interface/loader/gguf/gguf_reader.cpp:541-572, 678-724, 826-850).
//
// Design (HBM-bound: every weight byte is read exactly once, and the kernel
// spends as few instructions per byte as it can so that issue slots do not
// become the bound):
//  * Persistent CTAs own contiguous ranges of weight rows, walked in tiles of
//    16 rows.  The K axis of a tile is split over the CTA's warps.
//  * Each warp runs its own ring of shared-memory stages filled by bulk async
//    copies (cp.async.bulk, the TMA engine's untiled form; one copy per row
//    and stage, completion counted on an mbarrier).  A stage holds 16 rows x
//    256 or 512 weights of raw block bytes, row stride chosen so that the
//    fragment reads below are bank-conflict free.  A CTA's first copies are in
//    flight before it touches the activations.
//  * The 4- and 8-bit quants feed the integer tensor-core MMA directly
//    (m16n8k32, s8 x s8 -> s32): a nibble becomes the int8 value 16 (q - 8) with
//    one shift and one LOP3 per four weights, int8 quants are used as they
//    are.  18- and 34-byte blocks alternate between 4-byte aligned and
//    misaligned; blocks are consumed in aligned pairs with 32-bit loads, and
//    the k order inside a block is permuted per lane (the activations are
//    staged in the same permuted order), so no byte shuffling is needed.
//  * Activations are staged once per CTA as block floating point: per 32-k
//    block and activation row one fp32 scale e and 16-bit integers
//    x^ = rint(x / e), |x^| <= 32512, split into two balanced int8 digits that
//    occupy two MMA columns.  The integer dot product of a block is exact; it
//    is scaled by (fp16 block scale) x e in fp32 and accumulated in fp32.  fp16
//    activations keep ~16 bits relative to the block maximum (relative error of
//    a dot product ~3e-5); fp32 activations are staged as two such 16-bit
//    levels (32 bits).  Q4_K applies d*sc to the integer dot product and
//    dmin*m to the staged sum of x^, with the 6-bit fields unpacked in
//    registers.
//  * Partial sums of a CTA's warps meet in shared memory in a fixed order
//    (deterministic), then the fused epilogue runs and C is written.  With
//    ksplit > 1 (long K or few rows) partial sums go to a workspace and a
//    second small kernel adds them in a fixed order.
//
// Every wait on an mbarrier is bounded; on expiry the kernel stores
// CUTB_ERR_TIMEOUT in the caller's status word and leaves without spinning.
#include "common.cuh"
#include "kernels.h"

namespace cutb {

namespace {

constexpr int GV_ROWS = 16;

constexpr int GV_WARPS = 16;                      // consumer warps; one more warp issues the copies
constexpr int GV_THREADS = (GV_WARPS + 1) * 32;
constexpr int GV_KC = GV_WARPS;                   // granules (256 weights) per row and stage, one per consumer warp

// Shared-memory row stride of a stage (bytes): GV_KC granules plus the padding
// that keeps the 8 row groups of a warp on disjoint banks for the access
// pattern of the format (4 consecutive words per row for Q8_0 / Q4_0, 8 for Q4_K).
__host__ __device__ constexpr int gv_row_stride(int fmt) {
  return fmt == CUTB_Q8_0 ? 16 * 272 + 16    // 1092 words = 4 (mod 32)
         : fmt == CUTB_Q4_0 ? 16 * 144 + 16  // 580 words = 4 (mod 32)
                            : 16 * 144 + 32; // 584 words = 8 (mod 32)
}

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
  uint32_t stages;
  int fusion_type, fusion_op;
  int a_f32;
  int *status;
};

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
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

// int8 MMA, D = A * B with a zero accumulator (passed as four zero registers).
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Low / high nibbles of four bytes -> four int8 values 16 * (q - 8).
__device__ __forceinline__ uint32_t nib_lo_s(uint32_t x) { return ((x << 4) & 0xF0F0F0F0u) ^ 0x80808080u; }
__device__ __forceinline__ uint32_t nib_hi_s(uint32_t x) { return (x & 0xF0F0F0F0u) ^ 0x80808080u; }

// Element (0..31) of a 32-weight block that sits in byte i (0..7) of lane t's
// MMA fragment pair {b0, b1}; the weight side reads its bytes in the same
// order.  `even` = the block starts on a 4-byte boundary of the row.
template <int FMT> __device__ __forceinline__ uint32_t frag_elem(bool even, uint32_t t, uint32_t i) {
  if constexpr (FMT == CUTB_Q4_K) {
    return 8 * t + i;  // bytes 8t..8t+7 of the sub-block's 32 nibbles
  } else if constexpr (FMT == CUTB_Q4_0) {
    // byte index inside the 16 quant bytes; low nibble = element j, high = element j + 16
    const uint32_t j = i & 3;
    uint32_t byte;
    if (!even) byte = 4 * t + j;
    else if (t < 3) byte = 2 + 4 * t + j;
    else byte = (j < 2) ? j : 12 + j;  // {0, 1, 14, 15}
    return byte + ((i >> 2) << 4);
  } else {
    const uint32_t j = i & 3;
    if (!even) return (i < 4) ? 4 * t + j : 16 + 4 * t + j;
    if (i < 4) return 2 + 4 * t + j;
    if (t < 3) return 18 + 4 * t + j;
    return (j < 2) ? 30 + j : j - 2;  // {30, 31, 0, 1}
  }
}

// One stage of one warp: 16 rows x ngr granules of raw blocks at shared
// address `st`.  `actb` / `escb` / `sxb` point at the staged activations,
// scales and (Q4_K) scaled sums of the first 32-k block of the stage.
template <int FMT, int NT, int RS>
__device__ __forceinline__ void compute_stage(uint32_t st, uint32_t ngr, uint32_t actb, uint32_t act_stride,
                                              const uint32_t (&aoff)[NT], uint32_t escb, uint32_t sxb, uint32_t g,
                                              uint32_t t, float (&tot)[NT][2]) {
  constexpr uint32_t NV = NT * 4;
  const uint32_t rowA = st + g * RS, rowB = rowA + 8 * RS;

  // scale the exact integer block dot products and accumulate in fp32
  auto accumulate = [&](uint32_t kb, float dA, float dB, const uint32_t (&fa)[2], const uint32_t (&fb)[2]) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint2 x = lds_u64(actb + kb * act_stride + aoff[nt]);
      const float e = __uint_as_float(lds_u32(escb + (kb * NV + nt * 4 + t) * 4));
      int c[4];
      mma_s8(c, fa[0], fb[0], fa[1], fb[1], x.x, x.y);
      const float fg = (float)(c[0] * 256 + c[1]), fh = (float)(c[2] * 256 + c[3]);
      tot[nt][0] = fmaf(dA * e, fg, tot[nt][0]);
      tot[nt][1] = fmaf(dB * e, fh, tot[nt][1]);
    }
  };

  if constexpr (FMT == CUTB_Q4_0) {
    // pairs of 18-byte blocks = 9 aligned words: {d0,u0} {u1,u2} {u3,u4} {u5,u6} {u7,d1} {v0,v1} ... {v6,v7}
    const uint32_t o1 = (t == 3) ? 0u : 4u + 4u * t;
    const uint32_t selx = (t == 3) ? 0x5432u : 0x3210u;
    const uint32_t np = ngr * 4;
#pragma unroll 2
    for (uint32_t p = 0; p < np; ++p) {
      const uint32_t pa = rowA + p * 36, pb = rowB + p * 36;
      const uint32_t a0w = lds_u32(pa), a1w = lds_u32(pa + o1), a4w = lds_u32(pa + 16), a5w = lds_u32(pa + 20 + 4 * t);
      const uint32_t b0w = lds_u32(pb), b1w = lds_u32(pb + o1), b4w = lds_u32(pb + 16), b5w = lds_u32(pb + 20 + 4 * t);
      const uint32_t xa = __byte_perm(a1w, a4w, selx), xb = __byte_perm(b1w, b4w, selx);
      {
        const uint32_t fa[2] = {nib_lo_s(xa), nib_hi_s(xa)}, fb[2] = {nib_lo_s(xb), nib_hi_s(xb)};
        accumulate(2 * p, h2f_bits(a0w & 0xFFFFu), h2f_bits(b0w & 0xFFFFu), fa, fb);
      }
      {
        const uint32_t fa[2] = {nib_lo_s(a5w), nib_hi_s(a5w)}, fb[2] = {nib_lo_s(b5w), nib_hi_s(b5w)};
        accumulate(2 * p + 1, h2f_bits(a4w >> 16), h2f_bits(b4w >> 16), fa, fb);
      }
    }
  } else if constexpr (FMT == CUTB_Q8_0) {
    // pairs of 34-byte blocks = 17 aligned words: {d0,u0} {u1,u2} ... {u13,u14} {u15,d1} then 8 words of block 1
    const uint32_t selx = (t == 3) ? 0x7610u : 0x3210u;
    const uint32_t np = ngr * 4;
#pragma unroll 2
    for (uint32_t p = 0; p < np; ++p) {
      const uint32_t pa = rowA + p * 68, pb = rowB + p * 68;
      const uint32_t a0w = lds_u32(pa), a8w = lds_u32(pa + 32);
      const uint32_t b0w = lds_u32(pb), b8w = lds_u32(pb + 32);
      {
        const uint32_t fa[2] = {lds_u32(pa + 4 + 4 * t), __byte_perm(lds_u32(pa + 20 + 4 * t), a0w, selx)};
        const uint32_t fb[2] = {lds_u32(pb + 4 + 4 * t), __byte_perm(lds_u32(pb + 20 + 4 * t), b0w, selx)};
        accumulate(2 * p, h2f_bits(a0w & 0xFFFFu), h2f_bits(b0w & 0xFFFFu), fa, fb);
      }
      {
        const uint32_t fa[2] = {lds_u32(pa + 36 + 4 * t), lds_u32(pa + 52 + 4 * t)};
        const uint32_t fb[2] = {lds_u32(pb + 36 + 4 * t), lds_u32(pb + 52 + 4 * t)};
        accumulate(2 * p + 1, h2f_bits(a8w >> 16), h2f_bits(b8w >> 16), fa, fb);
      }
    }
  } else {  // Q4_K: ngr super-blocks of 144 bytes per row
    for (uint32_t s = 0; s < ngr; ++s) {
      const uint32_t pa = rowA + s * 144, pb = rowB + s * 144;
      const uint4 hA = lds_u128(pa), hB = lds_u128(pb);
      const float dA = h2f_bits(hA.x & 0xFFFFu), mA = h2f_bits(hA.x >> 16);
      const float dB = h2f_bits(hB.x & 0xFFFFu), mB = h2f_bits(hB.x >> 16);
      // 6-bit (scale, min) pairs, four sub-blocks per 32-bit word (gguf_reader.cpp:668-676)
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
          const float dsA = fmaf(dA, __uint_as_float(__byte_perm(scA[j >> 2], 0x4B000000u, sel)), ndA);
          const float dmA = fmaf(mA, __uint_as_float(__byte_perm(mnA[j >> 2], 0x4B000000u, sel)), nmA);
          const float dsB = fmaf(dB, __uint_as_float(__byte_perm(scB[j >> 2], 0x4B000000u, sel)), ndB);
          const float dmB = fmaf(mB, __uint_as_float(__byte_perm(mnB[j >> 2], 0x4B000000u, sel)), nmB);
          const uint32_t a0 = hi ? (qa.x >> 4) & 0x0F0F0F0Fu : qa.x & 0x0F0F0F0Fu;
          const uint32_t a2 = hi ? (qa.y >> 4) & 0x0F0F0F0Fu : qa.y & 0x0F0F0F0Fu;
          const uint32_t a1 = hi ? (qb.x >> 4) & 0x0F0F0F0Fu : qb.x & 0x0F0F0F0Fu;
          const uint32_t a3 = hi ? (qb.y >> 4) & 0x0F0F0F0Fu : qb.y & 0x0F0F0F0Fu;
          const uint32_t kb = s * 8 + j;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint2 x = lds_u64(actb + kb * act_stride + aoff[nt]);
            const uint32_t vi = (kb * NV + nt * 4 + t) * 4;
            const float e = __uint_as_float(lds_u32(escb + vi)), sx = __uint_as_float(lds_u32(sxb + vi));
            int c[4];
            mma_s8(c, a0, a1, a2, a3, x.x, x.y);
            const float fg = (float)(c[0] * 256 + c[1]), fh = (float)(c[2] * 256 + c[3]);
            tot[nt][0] = fmaf(dsA * e, fg, tot[nt][0]);
            tot[nt][1] = fmaf(dsB * e, fh, tot[nt][1]);
            tot[nt][0] = fmaf(-dmA, sx, tot[nt][0]);
            tot[nt][1] = fmaf(-dmB, sx, tot[nt][1]);
          }
        }
      }
    }
  }
}

template <bool AF32> __device__ __forceinline__ float load_act(const void *A, uint64_t idx) {
  if constexpr (AF32) return __ldg(reinterpret_cast<const float *>(A) + idx);
  return __half2float(__ldg(reinterpret_cast<const __half *>(A) + idx));
}

// Balanced int8 digits of |v| <= 32639: v = 256 * hi + lo, both in [-128, 127].
__device__ __forceinline__ void digits(int v, int &hi, int &lo) {
  lo = ((v + 128) & 0xFF) - 128;
  hi = (v - lo) >> 8;
}

constexpr float GV_QMAX = 32512.f;

// Stages the activations of blocks [0, nblk) of this K split (starting at k0)
// as two-digit block floating point in MMA fragment order.
//   act  : [blk][col][lane t][8 bytes]; col = 2 * vrow + digit (0 = high digit)
//   esc  : [blk][NV] fp32 scale of the integer dot product (includes the 1/16 of the Q4_0 nibble encoding)
//   sx   : [blk][NV] fp32 e * sum(x^) (Q4_K only)
template <int FMT, bool AF32, int NT, int THREADS>
__device__ __forceinline__ void stage_activations(const GvParams &p, uint8_t *act, float *esc, float *sx, uint32_t k0,
                                                  uint32_t nblk, uint32_t ncp, uint32_t tid) {
  constexpr uint32_t NV = NT * 4;
  const uint32_t nrows = p.M;
  const uint32_t nvr = AF32 ? 2 * nrows : nrows;
  const uint32_t nchunks = nblk * nrows * 4;
  const float wscale = (FMT == CUTB_Q4_0) ? 0.0625f : 1.0f;
  for (uint32_t base = 0; base < nchunks; base += THREADS) {  // uniform trip count: shuffles inside
    const uint32_t id = base + tid;
    const bool live = id < nchunks;
    const uint32_t ct = id & 3, q = id >> 2;
    const uint32_t m = live ? q % nrows : 0, kb = live ? q / nrows : 0;
    const bool even = (FMT == CUTB_Q4_K) || ((kb & 1) == 0);
    float x[8];
    float amax = 0.f;
    const uint64_t rowbase = (uint64_t)m * p.lda + k0 + kb * 32;
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
      x[i] = live ? load_act<AF32>(p.A, rowbase + frag_elem<FMT>(even, ct, i)) : 0.f;
      amax = fmaxf(amax, fabsf(x[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // a NaN anywhere in the block must surface: fmaxf drops NaNs, the sum does not
    float probe = ((x[0] + x[1]) + (x[2] + x[3])) + ((x[4] + x[5]) + (x[6] + x[7]));
    probe += __shfl_xor_sync(0xffffffffu, probe, 1);
    probe += __shfl_xor_sync(0xffffffffu, probe, 2);
    const bool finite = (amax < __int_as_float(0x7f800000)) && (probe == probe);
    const float inv = (amax > 0.f && finite) ? GV_QMAX / amax : 0.f;
    float e = finite ? amax * (1.0f / GV_QMAX) : __int_as_float(0x7fc00000);
    int v[8], isum = 0;
    uint32_t whi[2] = {0, 0}, wlo[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = __float2int_rn(x[i] * inv);
      isum += v[i];
      int hi, lo;
      digits(v[i], hi, lo);
      whi[i >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (i & 3));
      wlo[i >> 2] |= (uint32_t)(lo & 0xFF) << (8 * (i & 3));
    }
    const uint32_t vr = AF32 ? 2 * m : m;
    if constexpr (FMT == CUTB_Q4_K) {
      isum += __shfl_xor_sync(0xffffffffu, isum, 1);
      isum += __shfl_xor_sync(0xffffffffu, isum, 2);
    }
    if (live) {
      *reinterpret_cast<uint2 *>(act + ((size_t)(kb * ncp + 2 * vr) * 4 + ct) * 8) = make_uint2(whi[0], whi[1]);
      *reinterpret_cast<uint2 *>(act + ((size_t)(kb * ncp + 2 * vr + 1) * 4 + ct) * 8) = make_uint2(wlo[0], wlo[1]);
      if (ct == 0) {
        esc[kb * NV + vr] = e * wscale;
        if constexpr (FMT == CUTB_Q4_K) sx[kb * NV + vr] = e * (float)isum;
      }
    }
    if constexpr (AF32) {
      // second 16-bit level: the residual x - x^ e, at scale e / 65024
      const float e2 = e * (1.0f / (2.f * GV_QMAX)), inv2 = inv * (2.f * GV_QMAX);
      int isum2 = 0;
      uint32_t rhi[2] = {0, 0}, rlo[2] = {0, 0};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float r = fmaf(-(float)v[i], e, x[i]);
        const int w = __float2int_rn(r * inv2);
        isum2 += w;
        int hi, lo;
        digits(w, hi, lo);
        rhi[i >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (i & 3));
        rlo[i >> 2] |= (uint32_t)(lo & 0xFF) << (8 * (i & 3));
      }
      if constexpr (FMT == CUTB_Q4_K) {
        isum2 += __shfl_xor_sync(0xffffffffu, isum2, 1);
        isum2 += __shfl_xor_sync(0xffffffffu, isum2, 2);
      }
      if (live) {
        *reinterpret_cast<uint2 *>(act + ((size_t)(kb * ncp + 2 * vr + 2) * 4 + ct) * 8) = make_uint2(rhi[0], rhi[1]);
        *reinterpret_cast<uint2 *>(act + ((size_t)(kb * ncp + 2 * vr + 3) * 4 + ct) * 8) = make_uint2(rlo[0], rlo[1]);
        if (ct == 0) {
          esc[kb * NV + vr + 1] = e2 * wscale;
          if constexpr (FMT == CUTB_Q4_K) sx[kb * NV + vr + 1] = e2 * (float)isum2;
        }
      }
    }
  }
  // idle MMA columns read an all-zero column; idle virtual rows get scale 0
  const uint32_t ncols = 2 * nvr;
  if (ncp > ncols)
    for (uint32_t id = tid; id < nblk * 4; id += THREADS)
      *reinterpret_cast<uint2 *>(act + ((size_t)((id >> 2) * ncp + ncols) * 4 + (id & 3)) * 8) = make_uint2(0, 0);
  const uint32_t spare = NV - nvr;
  if (spare)
    for (uint32_t id = tid; id < nblk * spare; id += THREADS) {
      const uint32_t o = (id / spare) * NV + nvr + id % spare;
      esc[o] = 0.f;
      if constexpr (FMT == CUTB_Q4_K) sx[o] = 0.f;
    }
}

template <int FMT, bool AF32, int NT>
__global__ void __launch_bounds__(GV_THREADS, 1) qgemv_blocks_kernel(const GvParams p) {
  constexpr int RS = gv_row_stride(FMT);
  constexpr uint32_t GB = granule_bytes(FMT);
  constexpr uint32_t STAGE_BYTES = GV_ROWS * RS;
  constexpr uint32_t NV = NT * 4, NC8 = NT * 8;
  extern __shared__ __align__(128) uint8_t smem[];

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const uint32_t nvr = AF32 ? 2 * p.M : p.M;  // virtual activation rows (two per fp32 row)
  const uint32_t ncols = 2 * nvr;
  const uint32_t ncp = (ncols < NC8) ? ncols + 1 : ncols;
  const uint32_t nblk_alloc = p.gran_per_split * 8;
  const uint32_t S = p.stages;

  uint8_t *ring = smem;
  uint8_t *act = ring + (size_t)S * STAGE_BYTES;
  float *esc = reinterpret_cast<float *>(act + (size_t)nblk_alloc * ncp * 32);
  float *sx = esc + nblk_alloc * NV;
  float *red = sx + (FMT == CUTB_Q4_K ? nblk_alloc * NV : 0);  // two buffers of [GV_WARPS][16][NV]
  uint64_t *bars = reinterpret_cast<uint64_t *>(red + 2 * GV_WARPS * GV_ROWS * NV);  // full[S], empty[S]

  // rows of this CTA and granules (256 weights) of this K split; a stage holds
  // 16 rows x up to GV_KC granules, one granule per consumer warp
  const uint32_t r0 = (uint32_t)((uint64_t)blockIdx.x * p.N / gridDim.x);
  const uint32_t r1 = (uint32_t)((uint64_t)(blockIdx.x + 1) * p.N / gridDim.x);
  const uint32_t G = p.K >> 8;
  const uint32_t gs0 = blockIdx.y * p.gran_per_split;
  const uint32_t gs1 = min(G, gs0 + p.gran_per_split);
  const uint32_t ng = gs1 - gs0;
  const uint32_t cpt = (ng + GV_KC - 1) / GV_KC;  // K chunks (stages) per row tile
  const uint32_t ntiles = (r1 - r0 + GV_ROWS - 1) / GV_ROWS;
  const uint32_t total_stages = ntiles * cpt;

  const uint32_t ring_u = smem_u32(ring);
  const uint32_t full_u = smem_u32(bars), empty_u = full_u + S * 8;

  if (tid == 0) {
    for (uint32_t s = 0; s < S; ++s) {
      mbar_init(full_u + s * 8, 1);
      mbar_init(empty_u + s * 8, GV_WARPS);
    }
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == GV_WARPS) {
    // ---- producer warp: whole row segments, one bulk copy per row and stage ----
    bool dead = false;
    for (uint32_t j = 0; j < total_stages && !dead; ++j) {
      const uint32_t tile = j / cpt, c = j - tile * cpt, slot = j % S;
      if (j >= S) {
        const bool ok = mbar_wait_bounded(empty_u + slot * 8, ((j / S) - 1) & 1u);
        if (!__all_sync(0xffffffffu, ok)) {
          dead = true;
          if (lane == 0 && p.status) atomicExch(p.status, (int)CUTB_ERR_TIMEOUT);
          break;
        }
      }
      const uint32_t gq = gs0 + c * GV_KC;
      const uint32_t bytes = min((uint32_t)GV_KC, gs1 - gq) * GB;
      const uint32_t row_base = r0 + tile * GV_ROWS;
      const uint32_t valid = min((uint32_t)GV_ROWS, r1 - row_base);
      const uint32_t bar = full_u + slot * 8;
      if (lane == 0) mbar_arrive_expect_tx(bar, valid * bytes);
      __syncwarp();
      if (lane < valid)
        bulk_g2s(ring_u + slot * STAGE_BYTES + lane * RS, p.W + (uint64_t)(row_base + lane) * p.row_bytes + (uint64_t)gq * GB,
                 bytes, bar);
    }
    // stay resident until every copy issued here has landed (bounded)
    const uint32_t first = total_stages > S ? total_stages - S : 0;
    for (uint32_t j = first; j < total_stages; ++j) (void)mbar_wait_bounded(full_u + (j % S) * 8, (j / S) & 1u, 1u << 18);
    return;
  }

  // ---- consumer warps ---------------------------------------------------------
  stage_activations<FMT, AF32, NT, GV_WARPS * 32>(p, act, esc, sx, gs0 * 256, ng * 8, ncp, tid);
  asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");

  // per-lane activation fragment offsets (idle lanes read the zero column)
  uint32_t aoff[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const uint32_t col = nt * 8 + g;
    aoff[nt] = ((col < ncols ? col : ncols) * 4 + t) * 8;
  }
  const uint32_t act_u = smem_u32(act), act_stride = ncp * 32, esc_u = smem_u32(esc), sx_u = smem_u32(sx);

  bool dead = false;
  for (uint32_t tile = 0; tile < ntiles; ++tile) {
    float tot[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = 0.f;

    for (uint32_t c = 0; c < cpt; ++c) {
      const uint32_t j = tile * cpt + c, slot = j % S, parity = (j / S) & 1u;
      if (!dead) {
        const bool ok = mbar_wait_bounded(full_u + slot * 8, parity);
        if (!__all_sync(0xffffffffu, ok)) {
          dead = true;
          if (lane == 0 && p.status) atomicExch(p.status, (int)CUTB_ERR_TIMEOUT);
        }
      }
      const uint32_t gq = gs0 + c * GV_KC + warp;  // this warp's granule of the chunk
      if (!dead && gq < gs1) {
        const uint32_t kb0 = (gq - gs0) * 8;  // first 32-weight block of the granule inside the split
        compute_stage<FMT, NT, RS>(ring_u + slot * STAGE_BYTES + warp * GB, 1, act_u + kb0 * act_stride, act_stride, aoff,
                                   esc_u + kb0 * NV * 4, sx_u + kb0 * NV * 4, g, t, tot);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_u + slot * 8);
    }

    // meet the other warps' K slices in a fixed order (double-buffered: one barrier per tile)
    float *rbuf = red + (size_t)(tile & 1) * GV_WARPS * GV_ROWS * NV;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float *r = rbuf + ((size_t)warp * GV_ROWS) * NV + nt * 4 + t;
      r[g * NV] = tot[nt][0];
      r[(g + 8) * NV] = tot[nt][1];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");
    const uint32_t row_base = r0 + tile * GV_ROWS;
    for (uint32_t o = tid; o < GV_ROWS * p.M; o += GV_WARPS * 32) {
      const uint32_t row = o % GV_ROWS, m = o / GV_ROWS, n = row_base + row;
      if (n < r1) {
        float sum = 0.f;
        if constexpr (AF32) {
#pragma unroll
          for (int w = 0; w < GV_WARPS; ++w) {
            const float2 hl = *reinterpret_cast<const float2 *>(rbuf + ((size_t)w * GV_ROWS + row) * NV + 2 * m);
            sum += hl.x + hl.y;
          }
        } else {
#pragma unroll
          for (int w = 0; w < GV_WARPS; ++w) sum += rbuf[((size_t)w * GV_ROWS + row) * NV + m];
        }
        if (p.ksplit > 1) {
          p.partial[((size_t)blockIdx.y * p.M + m) * p.N + n] = sum;
        } else {
          const float dv = (p.fusion_type == CUTB_FUSION_BINARY) ? p.D[(size_t)m * p.ldd + n] : 0.f;
          p.C[(size_t)m * p.ldc + n] = apply_epilogue(sum, p.fusion_type, p.fusion_op, dv);
        }
      }
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

// ---- host side ---------------------------------------------------------------

struct GvPlan {
  uint32_t nt, nvr, ncp, grid_x, ksplit, gran_per_split, stages;
  size_t smem;
};

size_t gv_smem_bytes(int fmt, uint32_t stages, uint32_t nt, uint32_t ncp, uint32_t gran_per_split) {
  const size_t nblk = (size_t)gran_per_split * 8;
  size_t b = (size_t)stages * GV_ROWS * gv_row_stride(fmt);
  b += nblk * ncp * 32;
  b += nblk * nt * 4 * 4 * (fmt == CUTB_Q4_K ? 2 : 1);
  b += (size_t)2 * GV_WARPS * GV_ROWS * nt * 4 * 4;
  b += 2 * stages * 8;
  return b;
}

bool gv_plan(const cutb_qmatmul_desc &d, const DeviceInfo &di, GvPlan *pl) {
  const bool af32 = d.a_dtype == CUTB_F32;
  pl->nvr = af32 ? 2 * d.M : d.M;
  if (pl->nvr == 0 || pl->nvr > 16) return false;
  pl->nt = pl->nvr <= 4 ? 1 : (pl->nvr <= 8 ? 2 : 4);
  const uint32_t ncols = 2 * pl->nvr;
  pl->ncp = ncols < pl->nt * 8 ? ncols + 1 : ncols;
  const uint32_t G = d.K / 256;
  const uint32_t tiles = (d.N + GV_ROWS - 1) / GV_ROWS;
  pl->grid_x = tiles < (uint32_t)di.sm_count ? tiles : (uint32_t)di.sm_count;
  uint32_t want = 1;
  if (pl->grid_x * 2 <= (uint32_t)di.sm_count) want = (uint32_t)di.sm_count / pl->grid_x;
  if (want > G) want = G;
  const size_t limit = di.smem_optin;
  // deepest ring that fits; split K further only when two stages do not fit
  for (uint32_t ks = want; ks <= G; ++ks) {
    const uint32_t gps = (G + ks - 1) / ks;
    for (uint32_t st = 4; st >= 2; --st) {
      const size_t sm = gv_smem_bytes(d.format, st, pl->nt, pl->ncp, gps);
      if (sm <= limit) {
        pl->gran_per_split = gps;
        pl->ksplit = (G + gps - 1) / gps;
        pl->stages = st;
        pl->smem = sm;
        return true;
      }
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
  const uint32_t nvr = d.a_dtype == CUTB_F32 ? 2 * d.M : d.M;
  if (nvr > 16) return false;
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
  p.stages = pl.stages;
  p.fusion_type = d.fusion_type;
  p.fusion_op = d.fusion_op;
  p.a_f32 = af32;
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
