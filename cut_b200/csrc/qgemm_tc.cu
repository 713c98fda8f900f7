// Prefill GEMM over native GGUF blocks on the 5th-generation tensor cores.
//
// C[M, N] = epilogue(A[M, K] * dequant(W)^T), W = N rows of Q8_0 / Q4_0 / Q4_K
// blocks.  Replaces the reference's M > 1 tensor-core variants
// MatMulQ4CoopMatTiled / MatMulQ8CoopMatTiled (operators/impl/matmul/
// MatMulQ4CoopMatTiled.cu:7-125, MatMulQ8CoopMatTiled.cu:7-112), which stage
// fp16 tiles in shared memory for 16x8x16 mma.sync; numerically it follows them:
// activations and dequantised weights are rounded to fp16, products are
// accumulated in fp32.
//
// One CTA computes one 128 x 128 output tile with tcgen05.mma (kind::f16,
// M = 128, N = 128, K = 16 per instruction) accumulating in tensor memory:
//   warp 0      allocates 128 TMEM columns, then one elected lane issues the MMAs
//               of every K stage and commits them to the stage's "empty" barrier;
//   warps 1-4   stage the activation tile (fp16, or fp32 converted on the fly)
//               into shared memory in the K-major 128-byte-swizzled layout the
//               MMA reads, and afterwards run the epilogue: tcgen05.ld of the
//               accumulator, fused unary/binary op, stores to C;
//   warps 5-8   dequantise the weight tile: each thread owns one weight row,
//               reads its raw block bytes for the 64-k stage, widens the quants
//               to fp16 with half2 arithmetic (scale applied as in the
//               reference's tensor-core variants) and stores them in the same
//               swizzled layout.
// A 3-stage ring (32 KB per stage) lets two CTAs share an SM, so one CTA's
// epilogue overlaps the other's main loop.  The raster walks the M tiles of one
// weight tile back to back, so the raw weight bytes are served by L2 after
// their first use.
//
// Every wait is bounded; on expiry the CTA records CUTB_ERR_TIMEOUT in the
// caller's status word, skips its remaining work, frees its tensor memory and
// returns.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64;
constexpr int TC_STAGES = 3;
constexpr int TC_THREADS = 9 * 32;
constexpr uint32_t TC_TILE_BYTES = TC_BM * TC_BK * 2;  // 16 KB, A and B tiles alike
constexpr uint32_t TC_TMEM_COLS = 128;

struct TcParams {
  const uint8_t *W;
  uint64_t row_bytes;
  const void *A;
  uint32_t lda;
  float *C;
  uint32_t ldc;
  const float *D;
  uint32_t ldd;
  uint32_t M, K, N;
  int fusion_type, fusion_op;
  int a_f32;
  int *status;
};

// ---- tcgen05 / descriptor helpers ----------------------------------------------
// K-major operand tile, 64 fp16 (128 bytes) per row, 128-byte swizzle: rows are
// 128 bytes apart, groups of 8 rows 1024 bytes apart (the stride byte offset);
// the leading byte offset is unused for swizzled K-major layouts (encoded 1).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (ignored)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
// kind::f16 instruction descriptor: fp16 A and B, both K-major, fp32 accumulator.
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t m, uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Byte offset of 16-byte chunk `c` (0..7) of row `r` inside a swizzled tile.
__device__ __forceinline__ uint32_t sw128(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

__device__ __forceinline__ void st_chunk(uint8_t *tile, uint32_t r, uint32_t c, uint4 v) {
  *reinterpret_cast<uint4 *>(tile + sw128(r, c)) = v;
}

// four nibbles (low 4 bits of each byte of x) -> two half2 of exact integers
__device__ __forceinline__ void nib4_to_h2(uint32_t x, __half2 &h01, __half2 &h23) {
  const uint32_t m = x & 0x0F0F0F0Fu;
  const uint32_t p01 = __byte_perm(m, 0x64646464u, 0x4140), p23 = __byte_perm(m, 0x64646464u, 0x4342);  // 1024 + q
  const __half2 k1024 = __float2half2_rn(1024.f);
  h01 = __hsub2(u32_as_h2(p01), k1024);
  h23 = __hsub2(u32_as_h2(p23), k1024);
}
__device__ __forceinline__ void i8x4_to_h2(uint32_t x, __half2 &h01, __half2 &h23) {
  const uint32_t u = x ^ 0x80808080u;  // q + 128
  const uint32_t p01 = __byte_perm(u, 0x64646464u, 0x4140), p23 = __byte_perm(u, 0x64646464u, 0x4342);
  const __half2 k = __float2half2_rn(1152.f);
  h01 = __hsub2(u32_as_h2(p01), k);
  h23 = __hsub2(u32_as_h2(p23), k);
}

// Raw bytes of the 64 weights [k0, k0 + 64) of one row, as aligned 32-bit words:
// Q8_0 two 34-byte blocks (17 words), Q4_0 two 18-byte blocks (9 words), Q4_K the
// 16-byte super-block header and the 32 quant bytes of the 64-weight group (12 words).
// Loading is split from converting so that the next stage's bytes are in flight
// while this stage is converted.
template <int FMT> struct RawWords {
  static constexpr int N = FMT == CUTB_Q8_0 ? 17 : (FMT == CUTB_Q4_0 ? 9 : 12);
  uint32_t w[N];
};

template <int FMT> __device__ __forceinline__ void load_raw(const uint8_t *row, uint32_t k0, RawWords<FMT> &r) {
  if constexpr (FMT == CUTB_Q4_K) {
    const uint8_t *blk = row + (size_t)(k0 / 256) * 144;
    const uint32_t gq = (k0 % 256) / 64;
    const uint4 hd = __ldg(reinterpret_cast<const uint4 *>(blk));
    const uint4 q0 = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + 32 * gq));
    const uint4 q1 = __ldg(reinterpret_cast<const uint4 *>(blk + 32 + 32 * gq));
    r.w[0] = hd.x; r.w[1] = hd.y; r.w[2] = hd.z; r.w[3] = hd.w;
    r.w[4] = q0.x; r.w[5] = q0.y; r.w[6] = q0.z; r.w[7] = q0.w;
    r.w[8] = q1.x; r.w[9] = q1.y; r.w[10] = q1.z; r.w[11] = q1.w;
  } else {
    // a pair of 18- or 34-byte blocks starts on a 4-byte boundary (K is a multiple of 64)
    const uint32_t *p = reinterpret_cast<const uint32_t *>(row + (size_t)(k0 / 32) * block_bytes(FMT));
#pragma unroll
    for (int i = 0; i < RawWords<FMT>::N; ++i) r.w[i] = __ldg(p + i);
  }
}

// Dequantises the 64 weights held in `r` into 8 chunks of 8 halves (k order).
// Q8_0 / Q4_0 multiply the exact integer by the fp16 block scale in fp16, as the
// reference's tensor-core variants do (MatMulQ8CoopMatTiled.cu:71-74,
// MatMulQ4CoopMatTiled.cu:84-87); Q4_K applies fp16(d * sc) and fp16(dmin * m),
// the precision of the runner's affine re-encode (interface/runner/llama/llama.cpp:602-607).
template <int FMT> __device__ __forceinline__ void convert64(const RawWords<FMT> &r, uint32_t k0, uint4 (&out)[8]) {
  __half2 h[32];
  if constexpr (FMT == CUTB_Q8_0) {
    // words: {d0,q0,q1} {q2..q5} ... {q30,q31,d1} then block 1's 32 quants in 8 aligned words
    const __half2 d0 = __half2half2(__ushort_as_half((unsigned short)(r.w[0] & 0xFFFFu)));
    const __half2 d1 = __half2half2(__ushort_as_half((unsigned short)(r.w[8] >> 16)));
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      __half2 a, c;
      i8x4_to_h2(__funnelshift_r(r.w[w], r.w[w + 1], 16), a, c);  // quants 4w .. 4w+3 of block 0
      h[2 * w] = __hmul2(a, d0);
      h[2 * w + 1] = __hmul2(c, d0);
      i8x4_to_h2(r.w[9 + w], a, c);
      h[16 + 2 * w] = __hmul2(a, d1);
      h[16 + 2 * w + 1] = __hmul2(c, d1);
    }
  } else if constexpr (FMT == CUTB_Q4_0) {
    // words: {d0,b0,b1} {b2..b5} {b6..b9} {b10..b13} {b14,b15,d1} then block 1's 16 bytes in 4 aligned words
    const __half2 d0 = __half2half2(__ushort_as_half((unsigned short)(r.w[0] & 0xFFFFu)));
    const __half2 d1 = __half2half2(__ushort_as_half((unsigned short)(r.w[4] >> 16)));
    const __half2 k8 = __float2half2_rn(8.f);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const __half2 d = b ? d1 : d0;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t x = b ? r.w[5 + w] : __funnelshift_r(r.w[w], r.w[w + 1], 16);  // bytes 4w .. 4w+3
        __half2 a, c;
        nib4_to_h2(x, a, c);  // elements 4w .. 4w+3 (low nibbles)
        h[b * 16 + 2 * w] = __hmul2(__hsub2(a, k8), d);
        h[b * 16 + 2 * w + 1] = __hmul2(__hsub2(c, k8), d);
        nib4_to_h2(x >> 4, a, c);  // elements 16 + 4w .. (high nibbles)
        h[b * 16 + 8 + 2 * w] = __hmul2(__hsub2(a, k8), d);
        h[b * 16 + 8 + 2 * w + 1] = __hmul2(__hsub2(c, k8), d);
      }
    }
  } else {
    const uint32_t gq = (k0 % 256) / 64;  // 64-weight group: sub-blocks 2gq (low nibbles), 2gq + 1 (high)
    const float d = h2f_bits(r.w[0] & 0xFFFFu), dmin = h2f_bits(r.w[0] >> 16);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      // 6-bit scale / min of sub-block j (gguf_reader.cpp:668-676)
      const uint32_t j = 2 * gq + i, sh = 8 * (j & 3);
      const uint32_t lo_sc = (r.w[1] >> sh) & 0xFF, lo_mn = (r.w[2] >> sh) & 0xFF, hi = (r.w[3] >> sh) & 0xFF;
      const uint32_t sc = j < 4 ? (lo_sc & 63) : ((hi & 0xF) | ((lo_sc >> 6) << 4));
      const uint32_t mn = j < 4 ? (lo_mn & 63) : ((hi >> 4) | ((lo_mn >> 6) << 4));
      const __half2 ds = __float2half2_rn(d * (float)sc), dm = __float2half2_rn(-(dmin * (float)mn));
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        __half2 a, c;
        nib4_to_h2(r.w[4 + w] >> (4 * i), a, c);
        h[i * 16 + 2 * w] = __hfma2(a, ds, dm);
        h[i * 16 + 2 * w + 1] = __hfma2(c, ds, dm);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < 8; ++c)
    out[c] = make_uint4(h2_as_u32(h[4 * c]), h2_as_u32(h[4 * c + 1]), h2_as_u32(h[4 * c + 2]), h2_as_u32(h[4 * c + 3]));
}

template <int FMT>
__global__ void __launch_bounds__(TC_THREADS, 2) qgemm_tc_kernel(const TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // tiles must start on a 1024-byte boundary (the 128-byte swizzle repeats every 8 rows)
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *tileA = smem;                                   // [TC_STAGES][16 KB]
  uint8_t *tileB = smem + TC_STAGES * TC_TILE_BYTES;       // [TC_STAGES][16 KB]
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + 2 * TC_STAGES * TC_TILE_BYTES);  // full[S], empty[S], accum
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * TC_STAGES + 1);
  uint32_t *abort_flag = tmem_slot + 1;

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * TC_BN;
  const uint32_t nk = p.K / TC_BK;
  const uint32_t full_u = smem_u32(bars), empty_u = full_u + TC_STAGES * 8, accum_u = empty_u + TC_STAGES * 8;

  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(full_u + s * 8, 8);    // one arrival per loader / converter warp and stage
      mbar_init(empty_u + s * 8, 1);   // one tcgen05.commit per stage
    }
    mbar_init(accum_u, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    // one warp allocates the accumulator columns and publishes the TMEM base address
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TC_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto give_up = [&]() {
    if (p.status) atomicExch(p.status, (int)CUTB_ERR_TIMEOUT);
    atomicExch(abort_flag, 1u);
  };

  if (warp == 0) {
    // ---- MMA issuer ------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(TC_BM, TC_BN);
      bool dead = false;
      for (uint32_t ks = 0; ks < nk && !dead; ++ks) {
        const uint32_t s = ks % TC_STAGES;
        if (!mbar_wait_bounded(full_u + s * 8, (ks / TC_STAGES) & 1u)) {
          give_up();
          dead = true;
          break;
        }
        tc_fence_after();
        const uint64_t adesc = umma_desc_sw128(smem_u32(tileA + s * TC_TILE_BYTES));
        const uint64_t bdesc = umma_desc_sw128(smem_u32(tileB + s * TC_TILE_BYTES));
#pragma unroll
        for (uint32_t k4 = 0; k4 < TC_BK / 16; ++k4)  // 16 k = 32 bytes = 2 descriptor units along the swizzled row
          umma_f16(tmem_base, adesc + 2 * k4, bdesc + 2 * k4, idesc, (ks | k4) != 0);
        umma_commit(empty_u + s * 8);  // frees the stage when these MMAs have read it
      }
      if (!dead) umma_commit(accum_u);  // accumulator complete
    }
    __syncwarp();
  } else {
    // ---- producers: warps 1-4 stage the A tile, warps 5-8 dequantise W rows --------
    // Every thread keeps the next stage's bytes in flight (registers) while it
    // stores the current stage.  One lane per warp polls the "empty" barrier and
    // one lane per warp arrives on "full", so the barriers see 8 parties, not 256.
    const bool is_a = warp <= 4;
    const uint32_t pt = is_a ? tid - 32 : tid - 160;  // 0..127 within the producer group
    bool dead = false;
    auto acquire = [&](uint32_t ks) -> bool {  // warp-uniform: is stage ks free to be written?
      const uint32_t s = ks % TC_STAGES;
      uint32_t ok = 1;
      if (ks >= TC_STAGES && lane == 0) ok = mbar_wait_bounded(empty_u + s * 8, ((ks / TC_STAGES) - 1) & 1u) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) {
        if (lane == 0) give_up();
        dead = true;
      }
      return !dead && !*reinterpret_cast<volatile uint32_t *>(abort_flag);
    };
    auto release = [&](uint32_t ks) {
      fence_async_smem();  // make the generic-proxy stores visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(full_u + (ks % TC_STAGES) * 8);
    };
    if (is_a) {
      // thread -> 16-byte chunk (pt & 7) of rows (pt >> 3) + 16 i: eight lanes read one 128-byte row segment
      const uint32_t c = pt & 7, rb = pt >> 3;
      uint4 nxt[8];
      auto load_stage = [&](uint32_t ks) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t m = m0 + rb + 16 * i;
          nxt[i] = make_uint4(0, 0, 0, 0);
          if (m < p.M) {
            const size_t idx = (size_t)m * p.lda + (size_t)ks * TC_BK + 8 * c;
            if (p.a_f32) {
              const float *src = reinterpret_cast<const float *>(p.A) + idx;
              const float4 f0 = __ldg(reinterpret_cast<const float4 *>(src)), f1 = __ldg(reinterpret_cast<const float4 *>(src + 4));
              nxt[i] = make_uint4(h2_as_u32(__floats2half2_rn(f0.x, f0.y)), h2_as_u32(__floats2half2_rn(f0.z, f0.w)),
                                  h2_as_u32(__floats2half2_rn(f1.x, f1.y)), h2_as_u32(__floats2half2_rn(f1.z, f1.w)));
            } else {
              nxt[i] = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(p.A) + idx));
            }
          }
        }
      };
      load_stage(0);
      for (uint32_t ks = 0; ks < nk; ++ks) {
        uint4 out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = nxt[i];
        if (ks + 1 < nk) load_stage(ks + 1);
        if (!acquire(ks)) break;
        uint8_t *tile = tileA + (ks % TC_STAGES) * TC_TILE_BYTES;
#pragma unroll
        for (int i = 0; i < 8; ++i) st_chunk(tile, rb + 16 * i, c, out[i]);
        release(ks);
      }
    } else {
      const uint32_t r = pt, n = n0 + r;  // one weight row per thread
      const bool live = n < p.N;
      const uint8_t *wrow = p.W + (size_t)(live ? n : 0) * p.row_bytes;
      RawWords<FMT> nxt;
#pragma unroll
      for (int i = 0; i < RawWords<FMT>::N; ++i) nxt.w[i] = 0;
      if (live) load_raw<FMT>(wrow, 0, nxt);
      for (uint32_t ks = 0; ks < nk; ++ks) {
        const RawWords<FMT> cur = nxt;
        if (live && ks + 1 < nk) load_raw<FMT>(wrow, (ks + 1) * TC_BK, nxt);
        uint4 out[8];
        if (live) {
          convert64<FMT>(cur, ks * TC_BK, out);
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
        if (!acquire(ks)) break;
        uint8_t *tile = tileB + (ks % TC_STAGES) * TC_TILE_BYTES;
#pragma unroll
        for (int c = 0; c < 8; ++c) st_chunk(tile, r, c, out[c]);
        release(ks);
      }
    }

    // ---- epilogue: warps 1-4, one TMEM lane (= output row) per thread ---------------
    if (is_a && !dead && !*reinterpret_cast<volatile uint32_t *>(abort_flag)) {
      if (!mbar_wait_bounded(accum_u, 0)) {
        give_up();
      } else {
        tc_fence_after();
        const uint32_t q = warp & 3;  // TMEM lane quarter this warp may read
        const uint32_t row = q * 32 + lane;
        const uint32_t m = m0 + row;
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < TC_BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((q * 32) << 16) + c0, v);
          if (m < p.M) {
            float *dst = p.C + (size_t)m * p.ldc + n0 + c0;
            const float *dsrc = p.fusion_type == CUTB_FUSION_BINARY ? p.D + (size_t)m * p.ldd + n0 + c0 : nullptr;
            const bool vec = (n0 + c0 + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
            if (vec && p.fusion_type == CUTB_FUSION_NONE) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4 *>(dst)[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                                 __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n0 + c0 + i < p.N)
                  dst[i] = apply_epilogue(__uint_as_float(v[i]), p.fusion_type, p.fusion_op, dsrc ? dsrc[i] : 0.f);
            }
          }
        }
      }
    }
  }

  // release the tensor memory once every reader is done with it
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
  }
}

constexpr size_t TC_SMEM = 1024 + 2 * TC_STAGES * TC_TILE_BYTES + (2 * TC_STAGES + 1) * 8 + 16;

template <int FMT> int tc_launch(const TcParams &p, cudaStream_t stream) {
  static int configured_device = -1;
  int dev = 0;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    CUTB_CUDA_TRY(cudaFuncSetAttribute(qgemm_tc_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
    configured_device = dev;
  }
  // M tiles fastest: the CTAs that share a weight tile run back to back
  dim3 grid((p.M + TC_BM - 1) / TC_BM, (p.N + TC_BN - 1) / TC_BN);
  qgemm_tc_kernel<FMT><<<grid, TC_THREADS, TC_SMEM, stream>>>(p);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace

bool qgemm_tc_supported(const cutb_qmatmul_desc &d) {
  if (d.layout != CUTB_LAYOUT_GGUF_BLOCKS) return false;
  if (d.K == 0 || d.K % 256 != 0 || d.M == 0 || d.N == 0) return false;
  // 16-byte vector loads of the activation rows and of Q4_K super-blocks
  const uintptr_t a = reinterpret_cast<uintptr_t>(d.A), w = reinterpret_cast<uintptr_t>(d.W);
  if (a % 16 != 0 || w % 16 != 0) return false;
  if (d.a_dtype == CUTB_F32 ? d.lda % 4 != 0 : d.lda % 8 != 0) return false;
  DeviceInfo di;
  if (get_device_info(&di) != CUTB_OK) return true;  // shape check only (no device to ask)
  return di.cc_major == 10;
}

int qgemm_tc_launch(const cutb_qmatmul_desc &d, cudaStream_t stream) {
  TcParams p;
  p.W = reinterpret_cast<const uint8_t *>(d.W);
  p.row_bytes = row_bytes(d.format, d.K);
  p.A = d.A;
  p.lda = d.lda;
  p.C = d.C;
  p.ldc = d.ldc;
  p.D = d.D;
  p.ldd = d.ldd;
  p.M = d.M;
  p.K = d.K;
  p.N = d.N;
  p.fusion_type = d.fusion_type;
  p.fusion_op = d.fusion_op;
  p.a_f32 = d.a_dtype == CUTB_F32;
  p.status = d.status;
  switch (d.format) {
    case CUTB_Q8_0: return tc_launch<CUTB_Q8_0>(p, stream);
    case CUTB_Q4_0: return tc_launch<CUTB_Q4_0>(p, stream);
    default: return tc_launch<CUTB_Q4_K>(p, stream);
  }
}

}  // namespace cutb
