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
// One CTA owns one tile of 128 weight rows and up to 512 tokens, so a weight tile
// is dequantised once for all of them.  The weight tile is the MMA's M operand
// (one weight row per tensor-memory lane) and the tokens are its N operand, 256
// at a time: tcgen05.mma kind::f16 with M = 128, N = 256, K = 16 reads 12 KB of
// shared memory per instruction where the 128 x 128 shape reads 8 KB for half the
// work, and shared-memory bandwidth (operand reads + tile writes) is what bounds
// this kernel.  Each pair of 128-token blocks accumulates in its own 256 columns
// of tensor memory.
//   warp 0      allocates the TMEM columns; one lane issues the MMAs of every K stage
//               and commits them to the stage's "consumed" barrier, which frees both
//               the activation stage and the weight slot.  Its instruction stream is the kernel's critical
//               path (a lone thread retires an instruction every ~6 cycles), so the
//               loop keeps ring indices and descriptor words incrementally and
//               waits by polling, not by parking;
//   warp 2      a second issuer for the second token pair (independent accumulator);
//   warp 1      one lane issues the TMA tensor copies of the activation blocks
//               (64 k x 128 tokens of fp16, 128-byte swizzle, rows past M are
//               zero-filled by the copy engine), completion counted on the stage's
//               "full" barrier;
//   warps 4..   dequantise the weight tile in groups of four warps; group g owns the
//               K stages g, g + G, ...; each thread owns one weight row, keeps the
//               raw block bytes of its next stage in flight in registers, widens
//               the quants to fp16 with half2 arithmetic (scale applied as in the
//               reference's tensor-core variants) and stores them in the K-major
//               128-byte-swizzled layout the MMA reads; afterwards they run the
//               epilogue: tcgen05.ld of the accumulators (lane = weight row, column
//               = token), fused op, stores to C coalesced along n.
// fp32 activations are first rounded to fp16 into the caller's workspace by a
// small cast kernel (the copy engine cannot convert).  Shared memory holds a ring
// of activation stages (three at 512 tokens) and a ring of two weight tiles.
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

constexpr int TC_BW = 128;            // weight rows per CTA (MMA M, one per TMEM lane)
constexpr int TC_BT = 128;            // tokens per activation tile (rows of one TMA box)
constexpr int TC_BK = 64;             // k per stage: one 128-byte swizzled row of fp16
constexpr int TC_MAX_MB = 4;          // token blocks per CTA (4 x 128 columns = all of tensor memory)
constexpr int TC_MAX_GROUPS = 2;      // converter groups of 128 threads; group g dequantises K stages g, g + G, ...
constexpr int TC_CTRL_THREADS = 128;  // warps 0-3: issuer, copy producer, second issuer, spare
constexpr int TC_MAX_THREADS = TC_CTRL_THREADS + 128 * TC_MAX_GROUPS;
constexpr uint32_t TC_TILE_BYTES = 128 * TC_BK * 2;  // 16 KB: one token block, or the weight tile, per stage
constexpr uint32_t TC_TILE_DESC = TC_TILE_BYTES >> 4;  // the same in descriptor address units

struct TcParams {
  const uint8_t *W;
  uint64_t row_bytes;
  float *C;
  uint32_t ldc;
  const float *D;
  uint32_t ldd;
  uint32_t M, K, N;
  uint32_t mb;       // token blocks per CTA (1..4)
  uint32_t sa, nb;   // activation stages (of mb tiles each) and weight slots in shared memory
  uint32_t groups;   // converter groups (1..nb)
  uint32_t issuers;  // MMA issuer threads (1..2, at most one per token pair)
  uint32_t ksub;     // 64-k sub-tiles per stage (2 up to 256 tokens: the issuer's waits are paid per stage)
  int fusion_type, fusion_op;
  int *status;
  // the reference's [K, N] plane layout (TC_PLANE_* formats): value plane row stride in bytes, fp16 scale plane and its
  // row stride in elements, rows of the scale plane before the affine mins
  const uint16_t *S;
  uint32_t ldb, lds, blocksK;
};

// Weight sources of the converters besides the GGUF block formats: the reference's run-time planes
// (operators/impl/matmul/MatMulOp.cpp:309-329), int8 [K, ldb], nibbles [K, ldb] with even n in the low nibble,
// and the same with per-block mins behind the scales (the runner's affine re-encode of Q4_K).
constexpr int TC_PLANE_Q8 = 100, TC_PLANE_Q4 = 101, TC_PLANE_Q4A = 102;
__host__ __device__ constexpr bool tc_is_plane(int fmt) { return fmt >= TC_PLANE_Q8; }

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
// The descriptors of all tiles differ only in the start-address field, so the issuer keeps the
// low words and one shared high word; `accumulate` = 0 overwrites the accumulator.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint32_t adesc_lo, uint32_t bdesc_lo, uint32_t desc_hi, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(tmem_d), "r"(adesc_lo), "r"(bdesc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
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

// Raw bytes of the 64 weights [k0, k0 + 64) of one row, as 32-bit words: Q8_0 two
// 34-byte blocks (17 words), Q4_0 two 18-byte blocks (9 words), Q4_K the 16-byte
// super-block header and the 32 quant bytes of the 64-weight group (12 words).
template <int FMT> struct RawWords {
  static constexpr int N = FMT == CUTB_Q8_0 ? 17 : (FMT == CUTB_Q4_0 ? 9 : 12);
  uint32_t w[N];
};

// What a converter thread keeps in flight for its next stage: 16-byte loads only.  A
// thread per weight row means every lane of a load touches its own cache line, so the
// cost of a stage's loads is their count; the 68 (36) bytes of a Q8_0 (Q4_0) chunk start
// 0, 4, 8 or 12 bytes into a 16-byte line (k0 / 64 mod 4), and the aligned window of five
// (three) lines around them costs a third of the 17 (9) word loads.  Rows are a multiple
// of 16 bytes (K % 256 == 0) and the last chunk of a row ends on its last line, so the
// window never leaves the row.
template <int FMT> struct RawWindow {
  static constexpr int NV = FMT == CUTB_Q8_0 ? 5 : 3;
  uint4 v[NV];
};
// Plane layout: column n of 64 consecutive k rows is 64 separate bytes (a warp's 32 threads read 32 neighbouring
// bytes of one k row per load).  They are packed four quants to a word as they arrive -- int8 as stored, nibbles as
// one value per byte -- with the two block scales (and mins) of the 64 rows beside them.
template <> struct RawWindow<TC_PLANE_Q8> {
  static constexpr int NV = 4;
  uint4 v[NV];
  uint32_t sc;  // two f16 scales
};
template <> struct RawWindow<TC_PLANE_Q4> {
  static constexpr int NV = 4;
  uint4 v[NV];
  uint32_t sc;
};
template <> struct RawWindow<TC_PLANE_Q4A> {
  static constexpr int NV = 4;
  uint4 v[NV];
  uint32_t sc, mn;
};

template <int FMT> __device__ __forceinline__ void load_window_plane(const TcParams &p, uint32_t n, uint32_t k0, RawWindow<FMT> &r) {
  constexpr bool Q4 = FMT != TC_PLANE_Q8;
  const uint8_t *col = p.W + (size_t)k0 * p.ldb + (Q4 ? n >> 1 : n);
  const uint32_t shift = Q4 ? (n & 1u) * 4u : 0u;
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    uint32_t b[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = __ldg(col + (size_t)(4 * i + j) * p.ldb);
    if constexpr (Q4) {
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = (b[j] >> shift) & 0xFu;
    }
    w[i] = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
  const uint16_t *sp = p.S + (size_t)(k0 / 32) * p.lds + n;
  r.sc = (uint32_t)__ldg(sp) | ((uint32_t)__ldg(sp + p.lds) << 16);
  if constexpr (FMT == TC_PLANE_Q4A) {
    const uint16_t *mp = sp + (size_t)p.blocksK * p.lds;
    r.mn = (uint32_t)__ldg(mp) | ((uint32_t)__ldg(mp + p.lds) << 16);
  }
}

// 64 plane weights -> 8 chunks of 8 halves: the exact integer times the fp16 block scale in fp16 (plus the fp16 min),
// as the reference's tensor-core kernels widen them (MatMulQ8CoopMatTiled.cu:71-74, MatMulQ4CoopMatTiled.cu:84-87).
template <int FMT> __device__ __forceinline__ void convert_window_plane(const RawWindow<FMT> &win, uint4 (&out)[8]) {
  const uint32_t w[16] = {win.v[0].x, win.v[0].y, win.v[0].z, win.v[0].w, win.v[1].x, win.v[1].y, win.v[1].z, win.v[1].w,
                          win.v[2].x, win.v[2].y, win.v[2].z, win.v[2].w, win.v[3].x, win.v[3].y, win.v[3].z, win.v[3].w};
  const __half2 d0 = __half2half2(__ushort_as_half((unsigned short)(win.sc & 0xFFFFu)));
  const __half2 d1 = __half2half2(__ushort_as_half((unsigned short)(win.sc >> 16)));
  __half2 m0 = __float2half2_rn(0.f), m1 = m0;
  if constexpr (FMT == TC_PLANE_Q4A) {
    m0 = __half2half2(__ushort_as_half((unsigned short)(win.mn & 0xFFFFu)));
    m1 = __half2half2(__ushort_as_half((unsigned short)(win.mn >> 16)));
  }
  const __half2 k8 = __float2half2_rn(8.f);
  __half2 h[32];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const __half2 d = i < 8 ? d0 : d1;
    __half2 a, c;
    if constexpr (FMT == TC_PLANE_Q8) {
      i8x4_to_h2(w[i], a, c);
      h[2 * i] = __hmul2(a, d);
      h[2 * i + 1] = __hmul2(c, d);
    } else {
      nib4_to_h2(w[i], a, c);
      if constexpr (FMT == TC_PLANE_Q4A) {
        const __half2 m = i < 8 ? m0 : m1;
        h[2 * i] = __hfma2(__hsub2(a, k8), d, m);
        h[2 * i + 1] = __hfma2(__hsub2(c, k8), d, m);
      } else {
        h[2 * i] = __hmul2(__hsub2(a, k8), d);
        h[2 * i + 1] = __hmul2(__hsub2(c, k8), d);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < 8; ++c)
    out[c] = make_uint4(h2_as_u32(h[4 * c]), h2_as_u32(h[4 * c + 1]), h2_as_u32(h[4 * c + 2]), h2_as_u32(h[4 * c + 3]));
}

template <int FMT> __device__ __forceinline__ void load_window(const uint8_t *row, uint32_t k0, RawWindow<FMT> &r) {
  if constexpr (FMT == CUTB_Q4_K) {
    const uint8_t *blk = row + (size_t)(k0 / 256) * 144;
    const uint32_t gq = (k0 % 256) / 64;
    r.v[0] = __ldg(reinterpret_cast<const uint4 *>(blk));
    r.v[1] = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + 32 * gq));
    r.v[2] = __ldg(reinterpret_cast<const uint4 *>(blk + 32 + 32 * gq));
  } else {
    const size_t off = (size_t)(k0 / 32) * block_bytes(FMT);
    const uint4 *p = reinterpret_cast<const uint4 *>(row + (off & ~(size_t)15));
#pragma unroll
    for (int i = 0; i < RawWindow<FMT>::NV; ++i) r.v[i] = __ldg(p + i);
  }
}

// The chunk's words out of its window; S = (k0 / 64) % 4 is the chunk's word offset in
// the first line (static, so this is register renaming).
template <int FMT, int S> __device__ __forceinline__ void window_words(const RawWindow<FMT> &win, RawWords<FMT> &r) {
  uint32_t flat[RawWindow<FMT>::NV * 4];
#pragma unroll
  for (int i = 0; i < RawWindow<FMT>::NV; ++i) {
    flat[4 * i] = win.v[i].x;
    flat[4 * i + 1] = win.v[i].y;
    flat[4 * i + 2] = win.v[i].z;
    flat[4 * i + 3] = win.v[i].w;
  }
  constexpr int s = FMT == CUTB_Q4_K ? 0 : S;
#pragma unroll
  for (int i = 0; i < RawWords<FMT>::N; ++i) r.w[i] = flat[i + s];
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

template <int FMT> __device__ __forceinline__ void convert_window(const RawWindow<FMT> &win, uint32_t k0, uint4 (&out)[8]) {
  RawWords<FMT> r;
  if constexpr (FMT == CUTB_Q4_K) {
    window_words<FMT, 0>(win, r);
  } else {
    switch ((k0 / TC_BK) & 3u) {
      case 0: window_words<FMT, 0>(win, r); break;
      case 1: window_words<FMT, 1>(win, r); break;
      case 2: window_words<FMT, 2>(win, r); break;
      default: window_words<FMT, 3>(win, r); break;
    }
  }
  convert64<FMT>(r, k0, out);
}

template <int FMT>
__global__ void __launch_bounds__(TC_MAX_THREADS, 1) qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmapA, const TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // tiles must start on a 1024-byte boundary (the 128-byte swizzle repeats every 8 rows)
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t SA = p.sa, NB = p.nb, MB = p.mb, NI = p.issuers, KS = p.ksub;
  // a stage = KS sub-tiles of 64 k: activation tiles laid out [sub][token block], the weight slot [sub]
  const uint32_t a_stage_bytes = MB * KS * TC_TILE_BYTES, b_slot_bytes = KS * TC_TILE_BYTES;
  uint8_t *a_ring = smem, *b_ring = smem + SA * a_stage_bytes;
  // fullA[SA] fullB[NB] consumed[NC] accum.  One "consumed" barrier per K stage in a ring of
  // NC = SA + NB: a single tcgen05.commit per issuer and stage frees both the activation
  // stage and the weight slot (the copy producer waits for stage ks - SA, a converter for
  // stage ks - NB); NC > SA, NB keeps a barrier from being reused before both have seen it.
  const uint32_t NC = SA + NB;
  uint64_t *bars = reinterpret_cast<uint64_t *>(b_ring + NB * b_slot_bytes);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * SA + 2 * NB + 1);
  uint32_t *abort_flag = tmem_slot + 1;

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t n0 = blockIdx.x * TC_BW, m0 = blockIdx.y * (p.mb * TC_BT);
  const uint32_t nk = p.K / (TC_BK * KS);  // K stages
  const uint32_t fulla_u = smem_u32(bars), fullb_u = fulla_u + SA * 8, cons_u = fullb_u + NB * 8, accum_u = cons_u + NC * 8;
  const uint32_t tmem_cols = MB == 1 ? 128u : (MB == 2 ? 256u : 512u);

  if (tid == 0) {
    for (uint32_t s = 0; s < SA; ++s) mbar_init(fulla_u + s * 8, 1);  // the TMA lane's arrive.expect_tx
    for (uint32_t s = 0; s < NB; ++s) mbar_init(fullb_u + s * 8, 4);  // one arrival per converter warp of the owning group
    for (uint32_t s = 0; s < NC; ++s) mbar_init(cons_u + s * 8, NI);  // one tcgen05.commit per issuer and stage
    mbar_init(accum_u, NI);
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

  if (warp == 0 || warp == 2) {
    // ---- MMA issuers: issuer i owns the token pairs i, i + NI (256 tokens = 256 TMEM columns) ----
    const uint32_t me = warp >> 1;
    if (lane == 0 && me < NI) {
      const uint32_t npairs = (MB + 1) >> 1;
      // descriptor words: start address in the low word, stride / version / swizzle in the high word
      const uint64_t proto = umma_desc_sw128(0);
      const uint32_t desc_hi = (uint32_t)(proto >> 32), lo0 = (uint32_t)proto;
      const uint32_t w_lo0 = lo0 + ((smem_u32(b_ring) & 0x3FFFFu) >> 4), t_lo0 = lo0 + ((smem_u32(a_ring) & 0x3FFFFu) >> 4);
      const uint32_t idesc256 = umma_idesc_f16(TC_BW, 256), idesc128 = umma_idesc_f16(TC_BW, 128);
      uint32_t sa = 0, pa = 0, sb = 0, pb = 0, sc = 0;
      bool dead = false;
      for (uint32_t ks = 0; ks < nk; ++ks) {
        if (!mbar_spin_bounded(fullb_u + sb * 8, pb) || !mbar_spin_bounded(fulla_u + sa * 8, pa)) {
          give_up();
          dead = true;
          break;
        }
        tc_fence_after();
        for (uint32_t sub = 0; sub < KS; ++sub) {
          const uint32_t w_lo = w_lo0 + (sb * KS + sub) * TC_TILE_DESC, t_lo = t_lo0 + (sa * KS + sub) * MB * TC_TILE_DESC;
          const uint32_t acc = (ks | sub) != 0;
          for (uint32_t pr = me; pr < npairs; pr += NI) {
            const uint32_t idesc = (2 * pr + 2 <= MB) ? idesc256 : idesc128;
            const uint32_t tl = t_lo + pr * 2 * TC_TILE_DESC, d = tmem_base + pr * 256;
            // 16 k = 32 bytes = 2 descriptor units along the swizzled row
            umma_f16(d, w_lo, tl, desc_hi, idesc, acc);
            umma_f16(d, w_lo + 2, tl + 2, desc_hi, idesc, 1);
            umma_f16(d, w_lo + 4, tl + 4, desc_hi, idesc, 1);
            umma_f16(d, w_lo + 6, tl + 6, desc_hi, idesc, 1);
          }
        }
        umma_commit(cons_u + sc * 8);  // the stage is consumed when these MMAs have read it
        if (++sa == SA) sa = 0, pa ^= 1u;
        if (++sb == NB) sb = 0, pb ^= 1u;
        if (++sc == NC) sc = 0;
      }
      if (!dead) umma_commit(accum_u);  // this issuer's accumulators are complete
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- TMA producer: the activation blocks of every stage ------------------------------
    if (lane == 0) {
      uint32_t sa = 0, pa = 1u;  // parity of the slot's previous fill (used when draining)
      uint32_t sc = 0, pc = 0;   // consumed barrier of stage ks - SA
      uint32_t issued = 0;
      const uint32_t a_base = smem_u32(a_ring);
      for (uint32_t ks = 0; ks < nk; ++ks) {
        if (ks >= SA) {
          if (!mbar_spin_bounded(cons_u + sc * 8, pc)) {
            give_up();
            break;
          }
          if (++sc == NC) sc = 0, pc ^= 1u;
        }
        if (aborted()) break;
        const uint32_t bar = fulla_u + sa * 8, dst = a_base + sa * a_stage_bytes;
        mbar_arrive_expect_tx(bar, a_stage_bytes);
        for (uint32_t sub = 0; sub < KS; ++sub)
          for (uint32_t mb = 0; mb < MB; ++mb)
            tma_load_2d(dst + (sub * MB + mb) * TC_TILE_BYTES, &tmapA, (ks * KS + sub) * TC_BK, m0 + mb * TC_BT, bar);
        ++issued;
        if (++sa == SA) sa = 0, pa ^= 1u;
      }
      // an aborting CTA must not retire with copies still landing in its shared memory:
      // wait (bounded) for the last ring turn of copies it issued
      if (aborted()) {
        const uint32_t pending = issued < SA ? issued : SA;
        for (uint32_t i = 0; i < pending; ++i) {
          if (sa == 0) sa = SA, pa ^= 1u;
          --sa;
          mbar_wait_bounded(fulla_u + sa * 8, pa ^ 1u, 1u << 10);
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ---- converters: one weight row per thread; group g owns K stages g, g + G, ... and keeps
    // the raw bytes of its next stage in flight while it converts the current one (G <= NB) ----
    const uint32_t G = (blockDim.x - TC_CTRL_THREADS) >> 7;
    const uint32_t ct = tid - TC_CTRL_THREADS, r = ct & 127u, g = ct >> 7, n = n0 + r;
    const bool live = n < p.N;
    const uint8_t *wrow = tc_is_plane(FMT) ? p.W : p.W + (size_t)(live ? n : 0) * p.row_bytes;
    bool dead = false;
    RawWindow<FMT> nxt;
#pragma unroll
    for (int i = 0; i < RawWindow<FMT>::NV; ++i) nxt.v[i] = make_uint4(0, 0, 0, 0);
    if (live && g < nk) {
      if constexpr (tc_is_plane(FMT)) load_window_plane<FMT>(p, n, g * KS * TC_BK, nxt);
      else load_window<FMT>(wrow, g * KS * TC_BK, nxt);
    }
    // this group's slot sequence: start at slot g, advance by G modulo NB
    uint32_t sb = g % NB;
    uint32_t sc = 0, pc = 0;  // consumed barrier of stage ks - NB, once ks >= NB
    bool sc_set = false;
    for (uint32_t ks = g; ks < nk && !dead; ks += G) {
      uint8_t *slot = b_ring + sb * b_slot_bytes;
      for (uint32_t sub = 0; sub < KS; ++sub) {
        const uint32_t chunk = ks * KS + sub;  // 64-k chunk of the row
        const RawWindow<FMT> cur = nxt;
        // the chunk this thread converts next: the following sub-tile, or the first of the group's next stage
        const uint32_t nchunk = sub + 1 < KS ? chunk + 1 : (ks + G) * KS;
        if (live && nchunk < nk * KS) {
          if constexpr (tc_is_plane(FMT)) load_window_plane<FMT>(p, n, nchunk * TC_BK, nxt);
          else load_window<FMT>(wrow, nchunk * TC_BK, nxt);
        }
        uint4 out[8];
        if (live) {
          if constexpr (tc_is_plane(FMT)) convert_window_plane<FMT>(cur, out);
          else convert_window<FMT>(cur, chunk * TC_BK, out);
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
        if (sub == 0) {
          uint32_t ok = 1;  // one lane per warp polls the barrier
          if (ks >= NB) {
            if (!sc_set) sc = ks - NB, sc_set = true;  // first wait: stage ks - NB < G <= NB < NC
            if (lane == 0) ok = mbar_spin_bounded(cons_u + sc * 8, pc) ? 1u : 0u;
            sc += G;
            if (sc >= NC) sc -= NC, pc ^= 1u;
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) {
            if (lane == 0) give_up();
            dead = true;
          }
          if (dead || aborted()) {
            dead = true;
            break;
          }
        }
        uint8_t *tile = slot + sub * TC_TILE_BYTES;
#pragma unroll
        for (int c = 0; c < 8; ++c) st_chunk(tile, r, c, out[c]);
      }
      if (dead) break;
      fence_async_smem();  // make the generic-proxy stores visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(fullb_u + sb * 8);
      sb += G;
      if (sb >= NB) sb -= NB;  // G <= NB: at most one wrap
    }

    // ---- epilogue: one TMEM lane (= weight row) per thread, 32 token columns per item; the
    // groups share the items round-robin; a warp's stores of one token cover 32 consecutive n ----
    if (!dead && !aborted()) {
      if (!mbar_wait_bounded(accum_u, 0)) {
        give_up();
      } else {
        tc_fence_after();
        const uint32_t q = warp & 3;  // TMEM lane quarter this warp may read
        const uint32_t nn = n0 + q * 32 + lane;
        const bool n_ok = nn < p.N;
#pragma unroll 1
        for (uint32_t item = g; item < MB * (TC_BT / 32); item += G) {
          const uint32_t c0 = item * 32;  // token offset = accumulator column
          uint32_t v[32];
          tmem_ld32(tmem_base + ((q * 32) << 16) + c0, v);
          const uint32_t mbase = m0 + c0;
          if (mbase >= p.M) continue;
          float *dst = p.C + (size_t)mbase * p.ldc + nn;
          if (p.fusion_type == CUTB_FUSION_NONE) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n_ok && mbase + i < p.M) dst[(size_t)i * p.ldc] = __uint_as_float(v[i]);
          } else {
            const float *dsrc = p.fusion_type == CUTB_FUSION_BINARY ? p.D + (size_t)mbase * p.ldd + nn : nullptr;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n_ok && mbase + i < p.M)
                dst[(size_t)i * p.ldc] = apply_epilogue(__uint_as_float(v[i]), p.fusion_type, p.fusion_op,
                                                        dsrc ? dsrc[(size_t)i * p.ldd] : 0.f);
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

// fp32 activations -> fp16 rows of K elements (the TMA source of the GEMM).  A finite value beyond the
// fp16 range (it rounds to infinity) is reported through the caller's status word.
__global__ void cast_f32_f16_kernel(const float *__restrict__ A, uint32_t lda, __half *__restrict__ out, uint32_t M, uint32_t K,
                                    int *status) {
  const size_t total = (size_t)M * (K / 4);
  bool over = false;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / (K / 4), k = (i % (K / 4)) * 4;
    const float4 f = __ldg(reinterpret_cast<const float4 *>(A + m * lda + k));
    const float big = fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w)));  // NaN operands drop out of fmaxf
    over |= big > 65504.0f && big < __int_as_float(0x7f800000);
    *reinterpret_cast<uint2 *>(out + m * K + k) =
        make_uint2(h2_as_u32(__floats2half2_rn(f.x, f.y)), h2_as_u32(__floats2half2_rn(f.z, f.w)));
  }
  if (status && __any_sync(0xffffffffu, over) && (threadIdx.x & 31) == 0) atomicExch(status, (int)CUTB_ERR_RANGE);
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
  const cuuint32_t box[2] = {TC_BK, TC_BT};
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

size_t tc_smem_bytes(uint32_t mb, uint32_t sa, uint32_t nb, uint32_t ksub) {
  return 1024 + (size_t)(sa * mb + nb) * ksub * TC_TILE_BYTES + (2 * sa + 2 * nb + 1) * 8 + 16;  // fullA, fullB, consumed[sa + nb], accum
}

template <int FMT> int tc_launch(const CUtensorMap &map, const TcParams &p, cudaStream_t stream) {
  static bool configured[64] = {};  // per device: the attribute is set once on each
  int dev = 0;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    DeviceInfo di;
    if (int rc = get_device_info(&di)) return rc;
    CUTB_CUDA_TRY(cudaFuncSetAttribute(qgemm_tc_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)di.smem_optin));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid((p.N + TC_BW - 1) / TC_BW, (p.M + p.mb * TC_BT - 1) / (p.mb * TC_BT));
  qgemm_tc_kernel<FMT><<<grid, TC_CTRL_THREADS + 128 * p.groups, tc_smem_bytes(p.mb, p.sa, p.nb, p.ksub), stream>>>(map, p);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace

bool qgemm_tc_supported(const cutb_qmatmul_desc &d) {
  if (d.layout == CUTB_LAYOUT_KN_PLANES) {
    // the converters walk whole 128-row stages of the planes; the scale plane must hold K / 32 (or 2 K / 32) rows
    if (d.format != CUTB_Q8_0 && d.format != CUTB_Q4_0) return false;
    if (d.K == 0 || d.K % 128 != 0 || d.M == 0 || d.N == 0 || !d.scales) return false;
    const uint64_t row = d.format == CUTB_Q8_0 ? d.N : (d.N + 1) / 2;
    if (d.ldb < row || d.lds < d.N) return false;
  } else if (d.layout != CUTB_LAYOUT_GGUF_BLOCKS) {
    return false;
  }
  if (d.K == 0 || (d.layout == CUTB_LAYOUT_GGUF_BLOCKS && d.K % 256 != 0) || d.M == 0 || d.N == 0) return false;
  // 16-byte vector loads of the activation rows and of Q4_K super-blocks
  const uintptr_t a = reinterpret_cast<uintptr_t>(d.A), w = reinterpret_cast<uintptr_t>(d.W);
  if (a % 16 != 0 || (d.layout == CUTB_LAYOUT_GGUF_BLOCKS && w % 16 != 0)) return false;
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
  p.S = reinterpret_cast<const uint16_t *>(d.scales);
  p.ldb = d.ldb;
  p.lds = d.lds;
  p.blocksK = (d.K + 31) / 32;
  const uint32_t mblocks = (d.M + TC_BT - 1) / TC_BT;
  p.mb = mblocks < TC_MAX_MB ? mblocks : TC_MAX_MB;
  // Few weight rows (a 4096-row projection is 32 column tiles): fewer tokens per CTA until the grid covers at
  // least half of the SMs.  Each weight tile is then dequantised once per token group, which costs far less than
  // leaving three quarters of the SMs idle.
  {
    const uint32_t ctiles = (d.N + TC_BW - 1) / TC_BW;
    while (p.mb > 1 && ctiles * ((mblocks + p.mb - 1) / p.mb) * 2 <= (uint32_t)di.sm_count) p.mb = (p.mb + 1) / 2;
  }
  // two weight slots (one per converter group); the rest of shared memory holds activation
  // stages in flight
  p.nb = 2;
  p.groups = TC_MAX_GROUPS;
  if (p.groups > p.nb) p.groups = p.nb;
  p.issuers = 2;
  if (p.issuers > (p.mb + 1) / 2) p.issuers = (p.mb + 1) / 2;
  // Up to 256 tokens the tensor work of a 64-k stage (256-512 cycles) is less than what the issuer
  // thread spends on the stage's two barrier waits and four to eight MMA issues: stages of 128 k
  // halve the waits per k, and shared memory has room for them there.
  p.ksub = p.mb <= 2 ? 2u : 1u;
  p.sa = 0;
  for (uint32_t sa = 6; sa >= 2; --sa)
    if (tc_smem_bytes(p.mb, sa, p.nb, p.ksub) <= di.smem_optin) {
      p.sa = sa;
      break;
    }
  if (!p.sa) {
    set_last_error("qgemm: shared memory too small for the tile rings");
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
                                                    reinterpret_cast<__half *>(d.workspace), d.M, d.K, d.status);
    CUTB_CUDA_TRY(cudaGetLastError());
    a16 = d.workspace;
    stride = (uint64_t)d.K * sizeof(__half);
  }
  CUtensorMap map;
  if (int rc = make_tmap_a(&map, a16, d.M, d.K, stride)) return rc;
  if (d.layout == CUTB_LAYOUT_KN_PLANES) {
    if (d.format == CUTB_Q8_0) return tc_launch<TC_PLANE_Q8>(map, p, stream);
    return d.affine ? tc_launch<TC_PLANE_Q4A>(map, p, stream) : tc_launch<TC_PLANE_Q4>(map, p, stream);
  }
  switch (d.format) {
    case CUTB_Q8_0: return tc_launch<CUTB_Q8_0>(map, p, stream);
    case CUTB_Q4_0: return tc_launch<CUTB_Q4_0>(map, p, stream);
    default: return tc_launch<CUTB_Q4_K>(map, p, stream);
  }
}

}  // namespace cutb
