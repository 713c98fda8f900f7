// Shared pieces of the tcgen05 GEMM kernels over quantized weights: tile constants, UMMA / TMA / tensor-memory
// wrappers, the converters from raw GGUF blocks (or the reference's [K,N] planes) to fp16 operand tiles, the
// fp32 -> fp16 activation cast and the tensor-map encoder.  Included by the kernels' translation units only.
#pragma once
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
  int glu;  // rows in (gate, up) pairs: C[m, n / 2] = unary(acc[m, n]) * acc[m, n + 1], n even
  int *status;
  // the reference's [K, N] plane layout (TC_PLANE_* formats): value plane row stride in bytes, fp16 scale plane and its
  // row stride in elements, rows of the scale plane before the affine mins
  const uint16_t *S;
  uint32_t ldb, lds, blocksK;
  // long K on few weight rows: K stages shared out over blockIdx.z, partial sums [ksplit][M][N] in the workspace
  uint32_t ksplit;
  float *partial;
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
// (OFF = 8 gives q - 8 directly: 1024 + q and 1032 are both exact, so one subtraction does for two)
template <int OFF = 0> __device__ __forceinline__ void nib4_to_h2(uint32_t x, __half2 &h01, __half2 &h23) {
  const uint32_t m = x & 0x0F0F0F0Fu;
  const uint32_t p01 = __byte_perm(m, 0x64646464u, 0x4140), p23 = __byte_perm(m, 0x64646464u, 0x4342);  // 1024 + q
  const __half2 k = __float2half2_rn(1024.f + (float)OFF);
  h01 = __hsub2(u32_as_h2(p01), k);
  h23 = __hsub2(u32_as_h2(p23), k);
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

template <int FMT, class Params> __device__ __forceinline__ void load_window_plane(const Params &p, uint32_t n, uint32_t k0, RawWindow<FMT> &r) {
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
      nib4_to_h2<8>(w[i], a, c);  // q - 8
      if constexpr (FMT == TC_PLANE_Q4A) {
        const __half2 m = i < 8 ? m0 : m1;
        h[2 * i] = __hfma2(a, d, m);
        h[2 * i + 1] = __hfma2(c, d, m);
      } else {
        h[2 * i] = __hmul2(a, d);
        h[2 * i + 1] = __hmul2(c, d);
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
  #pragma unroll
    for (int b = 0; b < 2; ++b) {
      const __half2 d = b ? d1 : d0;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t x = b ? r.w[5 + w] : __funnelshift_r(r.w[w], r.w[w + 1], 16);  // bytes 4w .. 4w+3
        __half2 a, c;
        nib4_to_h2<8>(x, a, c);  // elements 4w .. 4w+3 (low nibbles), q - 8
        h[b * 16 + 2 * w] = __hmul2(a, d);
        h[b * 16 + 2 * w + 1] = __hmul2(c, d);
        nib4_to_h2<8>(x >> 4, a, c);  // elements 16 + 4w .. (high nibbles)
        h[b * 16 + 8 + 2 * w] = __hmul2(a, d);
        h[b * 16 + 8 + 2 * w + 1] = __hmul2(c, d);
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

int tc_encode_fn(EncodeTiledFn *out) {
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
  *out = encode;
  return CUTB_OK;
}

int make_tmap_a(CUtensorMap *map, const void *a_f16, uint32_t M, uint32_t K, uint64_t row_stride_bytes, uint32_t box_rows = TC_BT) {
  EncodeTiledFn encode = nullptr;
  if (int rc = tc_encode_fn(&encode)) return rc;
  const cuuint64_t dims[2] = {K, M};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {TC_BK, box_rows};
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

}  // namespace
}  // namespace cutb
