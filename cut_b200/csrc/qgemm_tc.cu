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
// One CTA owns one tile of 128 weight rows and up to four 128-token blocks
// (512 tokens) of the activations, so a weight tile is dequantised once for all
// of them.  tcgen05.mma (kind::f16, M = 128, N = 128, K = 16 per instruction)
// accumulates every token block in its own 128 columns of tensor memory:
//   warp 0      allocates the TMEM columns; one elected lane issues the MMAs of
//               every K stage (token blocks x 4 instructions) and commits them to
//               the stage's "empty" barrier;
//   warp 1      one lane issues the TMA tensor copies of the activation blocks
//               (64 k x 128 tokens of fp16, 128-byte swizzle, rows past M are
//               zero-filled by the copy engine), completion counted on the
//               stage's "full A" barrier;
//   warps 2-5   dequantise the weight tile: each thread owns one weight row, keeps
//               the next stage's raw block bytes in flight in registers, widens
//               the quants to fp16 with half2 arithmetic (scale applied as in the
//               reference's tensor-core variants) and stores them in the K-major
//               128-byte-swizzled layout the MMA reads; afterwards they run the
//               epilogue: tcgen05.ld of the accumulators, fused op, stores to C.
// fp32 activations are first rounded to fp16 into the caller's workspace by a
// small cast kernel (the copy engine cannot convert).  With four token blocks a
// stage is 80 KB and the ring has two stages; with fewer blocks it is deeper.
//
// Every wait is bounded; on expiry the CTA records CUTB_ERR_TIMEOUT in the
// caller's status word, skips its remaining work, frees its tensor memory and
// returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64;
constexpr int TC_MAX_MB = 4;          // token blocks per CTA (4 x 128 columns = all of tensor memory)
constexpr int TC_THREADS = 6 * 32;
constexpr uint32_t TC_TILE_BYTES = TC_BM * TC_BK * 2;  // 16 KB: one token block, or the weight tile, per stage

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
  uint32_t mb;      // token blocks per CTA (1..4)
  uint32_t stages;  // ring depth
  int fusion_type, fusion_op;
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
// 2-D TMA tile copy global -> this CTA's shared memory; x = innermost (k) coordinate in elements.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
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
__global__ void __launch_bounds__(TC_THREADS, 1) qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmapA, const TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // tiles must start on a 1024-byte boundary (the 128-byte swizzle repeats every 8 rows)
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t S = p.stages, MB = p.mb;
  const uint32_t stage_bytes = (MB + 1) * TC_TILE_BYTES;  // MB activation blocks, then the weight tile
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S * stage_bytes);  // fullA[S], fullB[S], empty[S], accum
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * S + 1);
  uint32_t *abort_flag = tmem_slot + 1;

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t n0 = blockIdx.x * TC_BN, m0 = blockIdx.y * (TC_MAX_MB * TC_BM);
  const uint32_t nk = p.K / TC_BK;
  const uint32_t fulla_u = smem_u32(bars), fullb_u = fulla_u + S * 8, empty_u = fullb_u + S * 8, accum_u = empty_u + S * 8;
  const uint32_t tmem_cols = MB == 1 ? 128u : (MB == 2 ? 256u : 512u);

  if (tid == 0) {
    for (uint32_t s = 0; s < S; ++s) {
      mbar_init(fulla_u + s * 8, 1);  // the TMA lane's arrive.expect_tx
      mbar_init(fullb_u + s * 8, 4);  // one arrival per converter warp
      mbar_init(empty_u + s * 8, 1);  // one tcgen05.commit per stage
    }
    mbar_init(accum_u, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
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
  auto aborted = [&]() { return *reinterpret_cast<volatile uint32_t *>(abort_flag) != 0; };

  if (warp == 0) {
    // ---- MMA issuer --------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(TC_BM, TC_BN);
      bool dead = false;
      for (uint32_t ks = 0; ks < nk && !dead; ++ks) {
        const uint32_t s = ks % S, par = (ks / S) & 1u;
        if (!mbar_wait_bounded(fulla_u + s * 8, par) || !mbar_wait_bounded(fullb_u + s * 8, par)) {
          give_up();
          dead = true;
          break;
        }
        tc_fence_after();
        const uint32_t stage_u = smem_u32(smem + s * stage_bytes);
        const uint64_t bdesc = umma_desc_sw128(stage_u + MB * TC_TILE_BYTES);
        for (uint32_t mb = 0; mb < MB; ++mb) {
          const uint64_t adesc = umma_desc_sw128(stage_u + mb * TC_TILE_BYTES);
#pragma unroll
          for (uint32_t k4 = 0; k4 < TC_BK / 16; ++k4)  // 16 k = 32 bytes = 2 descriptor units along the swizzled row
            umma_f16(tmem_base + mb * TC_BN, adesc + 2 * k4, bdesc + 2 * k4, idesc, (ks | k4) != 0);
        }
        umma_commit(empty_u + s * 8);  // frees the stage when these MMAs have read it
      }
      if (!dead) umma_commit(accum_u);  // accumulators complete
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- TMA producer: the activation blocks of every stage --------------------------
    if (lane == 0) {
      uint32_t issued = 0;
      for (uint32_t ks = 0; ks < nk; ++ks) {
        const uint32_t s = ks % S;
        if (ks >= S && !mbar_wait_bounded(empty_u + s * 8, ((ks / S) - 1) & 1u)) {
          give_up();
          break;
        }
        if (aborted()) break;
        const uint32_t bar = fulla_u + s * 8, dst = smem_u32(smem + s * stage_bytes);
        mbar_arrive_expect_tx(bar, MB * TC_TILE_BYTES);
        for (uint32_t mb = 0; mb < MB; ++mb) tma_load_2d(dst + mb * TC_TILE_BYTES, &tmapA, ks * TC_BK, m0 + mb * TC_BM, bar);
        ++issued;
      }
      // an aborting CTA must not retire with copies still landing in its shared memory
      if (aborted())
        for (uint32_t ks = issued > S ? issued - S : 0; ks < issued; ++ks) mbar_wait_bounded(fulla_u + (ks % S) * 8, (ks / S) & 1u, 1u << 10);
    }
    __syncwarp();
  } else {
    // ---- converters: one weight row per thread, next stage's bytes kept in flight -------
    const uint32_t r = tid - 64, n = n0 + r;
    const bool live = n < p.N;
    const uint8_t *wrow = p.W + (size_t)(live ? n : 0) * p.row_bytes;
    bool dead = false;
    RawWords<FMT> nxt;
#pragma unroll
    for (int i = 0; i < RawWords<FMT>::N; ++i) nxt.w[i] = 0;
    if (live) load_raw<FMT>(wrow, 0, nxt);
    for (uint32_t ks = 0; ks < nk; ++ks) {
      const uint32_t s = ks % S;
      const RawWords<FMT> cur = nxt;
      if (live && ks + 1 < nk) load_raw<FMT>(wrow, (ks + 1) * TC_BK, nxt);
      uint4 out[8];
      if (live) {
        convert64<FMT>(cur, ks * TC_BK, out);
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) out[c] = make_uint4(0, 0, 0, 0);
      }
      uint32_t ok = 1;  // one lane per warp polls the barrier
      if (ks >= S && lane == 0) ok = mbar_wait_bounded(empty_u + s * 8, ((ks / S) - 1) & 1u) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) {
        if (lane == 0) give_up();
        dead = true;
      }
      if (dead || aborted()) break;
      uint8_t *tile = smem + s * stage_bytes + MB * TC_TILE_BYTES;
#pragma unroll
      for (int c = 0; c < 8; ++c) st_chunk(tile, r, c, out[c]);
      fence_async_smem();  // make the generic-proxy stores visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(fullb_u + s * 8);
    }

    // ---- epilogue: one TMEM lane (= token row of each block) per thread --------------------
    if (!dead && !aborted()) {
      if (!mbar_wait_bounded(accum_u, 0)) {
        give_up();
      } else {
        tc_fence_after();
        const uint32_t q = warp & 3;  // TMEM lane quarter this warp may read
        for (uint32_t mb = 0; mb < MB; ++mb) {
          const uint32_t m = m0 + mb * TC_BM + q * 32 + lane;
#pragma unroll 1
          for (uint32_t c0 = 0; c0 < TC_BN; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_base + ((q * 32) << 16) + mb * TC_BN + c0, v);
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
  }

  // release the tensor memory once every reader is done with it
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// fp32 activations -> fp16 rows of K elements (the TMA source of the GEMM)
__global__ void cast_f32_f16_kernel(const float *__restrict__ A, uint32_t lda, __half *__restrict__ out, uint32_t M, uint32_t K) {
  const size_t total = (size_t)M * (K / 4);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / (K / 4), k = (i % (K / 4)) * 4;
    const float4 f = __ldg(reinterpret_cast<const float4 *>(A + m * lda + k));
    *reinterpret_cast<uint2 *>(out + m * K + k) =
        make_uint2(h2_as_u32(__floats2half2_rn(f.x, f.y)), h2_as_u32(__floats2half2_rn(f.z, f.w)));
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tmap_a(CUtensorMap *map, const void *a_f16, uint32_t M, uint32_t K, uint64_t row_stride_bytes) {
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    CUTB_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess) {
      set_last_error("qgemm: the driver does not provide cuTensorMapEncodeTiled");
      return CUTB_ERR_CUDA;
    }
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const cuuint64_t dims[2] = {K, M};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {TC_BK, TC_BM};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a_f16), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("qgemm: cuTensorMapEncodeTiled failed with %d (M=%u K=%u stride=%llu)", (int)r, M, K,
                   (unsigned long long)row_stride_bytes);
    return CUTB_ERR_CUDA;
  }
  return CUTB_OK;
}

size_t tc_smem_bytes(uint32_t mb, uint32_t stages) {
  return 1024 + (size_t)stages * (mb + 1) * TC_TILE_BYTES + (3 * stages + 1) * 8 + 16;
}

template <int FMT> int tc_launch(const CUtensorMap &map, const TcParams &p, cudaStream_t stream) {
  static int configured_device = -1;
  int dev = 0;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_device != dev) {
    DeviceInfo di;
    if (int rc = get_device_info(&di)) return rc;
    CUTB_CUDA_TRY(cudaFuncSetAttribute(qgemm_tc_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)di.smem_optin));
    configured_device = dev;
  }
  dim3 grid((p.N + TC_BN - 1) / TC_BN, (p.M + TC_MAX_MB * TC_BM - 1) / (TC_MAX_MB * TC_BM));
  qgemm_tc_kernel<FMT><<<grid, TC_THREADS, tc_smem_bytes(p.mb, p.stages), stream>>>(map, p);
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

uint64_t qgemm_tc_workspace(const cutb_qmatmul_desc &d) {
  // fp32 activations are rounded to fp16 rows of K elements first
  return d.a_dtype == CUTB_F32 ? (uint64_t)d.M * d.K * sizeof(__half) : 0;
}

int qgemm_tc_launch(const cutb_qmatmul_desc &d, cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
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
  p.status = d.status;
  const uint32_t mblocks = (d.M + TC_BM - 1) / TC_BM;
  p.mb = mblocks < TC_MAX_MB ? mblocks : TC_MAX_MB;
  p.stages = 0;
  for (uint32_t st = 6; st >= 2; --st)
    if (tc_smem_bytes(p.mb, st) <= di.smem_optin) {
      p.stages = st;
      break;
    }
  if (!p.stages) {
    set_last_error("qgemm: shared memory too small for a two-stage ring");
    return CUTB_ERR_UNSUPPORTED;
  }
  const void *a16 = d.A;
  uint64_t stride = (uint64_t)d.lda * sizeof(__half);
  if (d.a_dtype == CUTB_F32) {
    const uint64_t need = qgemm_tc_workspace(d);
    if (!d.workspace || d.workspace_bytes < need || reinterpret_cast<uintptr_t>(d.workspace) % 16 != 0) {
      set_last_error("qgemm: fp32 activations need %llu bytes of 16-byte aligned workspace, got %llu",
                     (unsigned long long)need, (unsigned long long)d.workspace_bytes);
      return CUTB_ERR_WORKSPACE;
    }
    const size_t total = (size_t)d.M * (d.K / 4);
    const unsigned blocks = (unsigned)((total + 255) / 256 < (size_t)di.sm_count * 8 ? (total + 255) / 256 : (size_t)di.sm_count * 8);
    cast_f32_f16_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float *>(d.A), d.lda,
                                                    reinterpret_cast<__half *>(d.workspace), d.M, d.K);
    CUTB_CUDA_TRY(cudaGetLastError());
    a16 = d.workspace;
    stride = (uint64_t)d.K * sizeof(__half);
  }
  CUtensorMap map;
  if (int rc = make_tmap_a(&map, a16, d.M, d.K, stride)) return rc;
  switch (d.format) {
    case CUTB_Q8_0: return tc_launch<CUTB_Q8_0>(map, p, stream);
    case CUTB_Q4_0: return tc_launch<CUTB_Q4_0>(map, p, stream);
    default: return tc_launch<CUTB_Q4_K>(map, p, stream);
  }
}

}  // namespace cutb
