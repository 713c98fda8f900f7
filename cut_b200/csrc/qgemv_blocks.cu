// Decode mat-vec (a few activation rows) over native GGUF blocks for sm_100a.
//
// C[m, n] = sum_k A[m, k] * dequant(W)[n, k], W = N rows of Q8_0 / Q4_0 / Q4_K
// blocks.  Replaces the reference's M = 1 variants MatMulQ4GemvKPar8 /
// MatMulQ8GemvKPar8 (operators/impl/matmul/MatMulQ4GemvKPar8.cu:8-98,
// MatMulQ8GemvKPar8.cu:11-92) on the block layout its loader reads
// (interface/loader/gguf/gguf_reader.cpp:541-572, 678-724, 826-850).
//
// Design (every weight byte is read from DRAM exactly once, and the kernel spends as few
// instructions per byte as it can so that issue slots do not become the bound):
//  * One persistent CTA per SM owns a contiguous range of weight rows, walked in tiles of
//    16 rows.  A producer warp fills a ring of shared-memory stages with bulk async copies
//    (cp.async.bulk, the TMA engine's untiled form): one copy per row and stage of the whole
//    row segment (up to 4096 weights: 2304 bytes for the 4-bit formats, 4352 for Q8_0 --
//    large contiguous reads keep DRAM pages open), completion counted on an mbarrier.  The
//    K axis of a stage is split over 16 consumer warps, one 256-weight granule each; row
//    strides in shared memory are padded so that the fragment reads are bank-conflict free.
//    Q8_0 stages have a barrier pair per K half, so that half a stage can be refilled while
//    the other half is still being read.
//  * The kernel is launched with programmatic stream serialization: it lets its successor
//    start at once (griddepcontrol.launch_dependents), issues its first copies, and waits for
//    its predecessor (griddepcontrol.wait) only before it reads the activations; the
//    shared-memory plan keeps a CTA under half an SM so that both launches' CTAs co-reside.
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
//    (deterministic), then the fused epilogue runs and C is written (or, for a
//    row-sharded launch, stored into every rank's output through peer-mapped
//    pointers).  With ksplit > 1 (long K or few rows) partial sums go to a
//    workspace and a second small kernel adds them in a fixed order.
//
// Every wait on an mbarrier is bounded; on expiry the kernel stores
// CUTB_ERR_TIMEOUT in the caller's status word and leaves without spinning.
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace cutb {

namespace {

constexpr int GV_ROWS = 16;

constexpr int GV_WARPS = 16;                      // consumer warps; one more warp issues the copies
constexpr int GV_THREADS = (GV_WARPS + 1) * 32;
// how the activations are read and staged
constexpr int GV_A_HALF = 0, GV_A_F32_TWO = 1, GV_A_F32_ONE = 2;

constexpr int GV_KC = GV_WARPS;                   // granules (256 weights) per row and stage, one per consumer warp

// Shared-memory layout of a stage: the 16 rows of a tile sit in 8 pairs, tile rows 2i and 2i + 1
// back to back (one full row segment of GV_KC granules each), pairs GV pair-stride bytes apart.
// MMA row g reads tile row 2g and MMA row g + 8 reads tile row 2g + 1 -- in different load
// instructions, so the two rows of a pair may share banks, while the padding of the pair stride
// keeps the 8 pairs of one instruction on disjoint banks (4 consecutive words per row for Q8_0 /
// Q4_0 and the Q4_K diagonal variant, 8 for Q4_K shared-k).  Two rows that are adjacent in global
// memory thus land adjacent in shared memory: when a stage holds whole rows, one bulk copy moves
// a pair (the copy engine takes about as long to accept a copy whatever its size).
__host__ __device__ constexpr int gv_raw_row(int fmt) { return GV_KC * (fmt == CUTB_Q8_0 ? 272 : 144); }
__host__ __device__ constexpr int gv_pair_stride(int fmt, bool diag) {
  return 2 * gv_raw_row(fmt) + ((fmt == CUTB_Q4_K && !diag) ? 32 : 16);  // = 4 or 8 words (mod 32)
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
  int glu;              // rows in (gate, up) pairs: C[m, i] = unary(acc[2i]) * acc[2i + 1]
  const float *norm_w;  // fused RMSNorm of the activation rows (nullptr: none)
  float norm_eps;
  int *status;
  // Activations staged once for all CTAs by stage_acts_kernel (nullptr: every CTA stages its own):
  // one blob per K split in the shared-memory layout [act | esc | sx], staged_bytes each.
  uint8_t *staged;
  uint32_t staged_bytes;
  // Row-sharded scatter epilogue (world > 1): instead of C, the output slice is stored into
  // every rank's full output at column n_off.  Peer-mapped pointers; plain stores, no
  // multicast, no fence here: the step's exchange kernel publishes them.
  uint32_t world, n_off, ldc_total;
  float *peer_C[CUTB_MAX_PEERS];
};

// Shared-memory loads by 32-bit shared address.  Plain loads through an
// address-space-qualified pointer rather than inline asm, so the compiler can
// schedule them freely between the (memory-clobbering) barrier waits.
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  return *reinterpret_cast<const uint32_t *>(__cvta_shared_to_generic(addr));
}
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
  return *reinterpret_cast<const uint2 *>(__cvta_shared_to_generic(addr));
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
  return *reinterpret_cast<const uint4 *>(__cvta_shared_to_generic(addr));
}

// int8 MMA, D = A * B with a zero accumulator.  UA: the A operand holds unsigned bytes.
template <bool UA>
__device__ __forceinline__ void mma_i8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  if constexpr (UA)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// int8 MMA accumulating into d.
template <bool UA>
__device__ __forceinline__ void mma_i8_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  if constexpr (UA)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Low / high nibbles of four bytes -> four unsigned bytes 16 * q.  The Q4_0
// offset (q - 8) is applied after the MMA through the staged sum of the
// activations of the block: sum((q - 8) x) = sum(q x) - 8 sum(x).
__device__ __forceinline__ uint32_t nib_lo_s(uint32_t x) { return (x << 4) & 0xF0F0F0F0u; }
__device__ __forceinline__ uint32_t nib_hi_s(uint32_t x) { return x & 0xF0F0F0F0u; }

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

// "Diagonal" variant used for one or two activation rows.  Lane t of a quad owns
// whole blocks (2t and 2t+1 of each 8-block granule) instead of a quarter of
// every block; its activation column pair is non-zero only in its own k slots,
// so MMA column pair t ends up holding the dot product of the lane's own block:
// the block scale is then applied once per block by the lane that loaded it.
// Element of a 32-weight block in byte b (0..7) of the fragment of MMA i (0..3).
template <int FMT> __device__ __forceinline__ uint32_t diag_elem(bool even, uint32_t i, uint32_t b) {
  const uint32_t j = b & 3;
  if constexpr (FMT == CUTB_Q4_K) {
    return 8 * i + b;
  } else if constexpr (FMT == CUTB_Q4_0) {
    uint32_t byte;
    if (!even) byte = 4 * i + j;
    else if (i < 3) byte = 2 + 4 * i + j;
    else byte = (j < 2) ? j : 12 + j;  // {0, 1, 14, 15}
    return byte + ((b >> 2) << 4);
  } else {
    const uint32_t w = 2 * i + (b >> 2);
    if (!even) return 4 * w + j;
    if (w < 7) return 2 + 4 * w + j;
    return (j < 2) ? j : 28 + j;  // {0, 1, 30, 31}
  }
}

// The four MMAs of one block in two independent accumulation chains.  r0* / r1*:
// first and second A register of MMA i for rows g (a) and g + 8 (b); act: shared
// address of the lane's 32 staged activation bytes of the block.
template <bool UA>
__device__ __forceinline__ void block_mmas(int (&c)[4], int (&c2)[4], const uint32_t (&r0a)[4], const uint32_t (&r0b)[4],
                                           const uint32_t (&r1a)[4], const uint32_t (&r1b)[4], uint32_t act) {
  const uint4 x0 = lds_u128(act), x1 = lds_u128(act + 16);
  mma_i8<UA>(c, r0a[0], r0b[0], r1a[0], r1b[0], x0.x, x0.y);
  mma_i8<UA>(c2, r0a[1], r0b[1], r1a[1], r1b[1], x0.z, x0.w);
  mma_i8_acc<UA>(c, r0a[2], r0b[2], r1a[2], r1b[2], x1.x, x1.y);
  mma_i8_acc<UA>(c2, r0a[3], r0b[3], r1a[3], r1b[3], x1.z, x1.w);
}

// One granule (8 blocks of 32 weights, or one Q4_K super-block) x 16 rows for
// the diagonal variant.  `rowA`: shared address of row g's granule; actp/escp/sxp:
// per-lane shared addresses of the lane's even block (see the kernel), pass_a /
// pass_e: byte distance to its odd block (0 for lanes whose columns are idle).
template <int FMT, int NVR>
__device__ __forceinline__ void compute_granule_diag(uint32_t rowA, const uint32_t (&actp)[NVR], uint32_t pass_a,
                                                     const uint32_t (&escp)[NVR], const uint32_t (&sxp)[NVR],
                                                     uint32_t pass_e, uint32_t t, float (&tot)[NVR][2]) {
  const uint32_t rowB = rowA + gv_raw_row(FMT);  // the pair's second row: MMA row g + 8
  // c / c2: two independent accumulation chains of the block's four MMAs
  auto finish = [&](int nt, const int (&c)[4], const int (&c2)[4], float sA, float sB, uint32_t eoff) {
    const float e = __uint_as_float(lds_u32(escp[nt] + eoff));
    const float fg = (float)((c[0] + c2[0]) * 256 + (c[1] + c2[1])), fh = (float)((c[2] + c2[2]) * 256 + (c[3] + c2[3]));
    if constexpr (FMT == CUTB_Q4_0) {
      // d * (e/16 * sum(16 q x^) - 8 e sum(x^)) = d e sum((q - 8) x^)
      const float off = __uint_as_float(lds_u32(sxp[nt] + eoff));
      tot[nt][0] = fmaf(sA, fmaf(e, fg, -off), tot[nt][0]);
      tot[nt][1] = fmaf(sB, fmaf(e, fh, -off), tot[nt][1]);
    } else {
      tot[nt][0] = fmaf(sA * e, fg, tot[nt][0]);
      tot[nt][1] = fmaf(sB * e, fh, tot[nt][1]);
    }
  };
  if constexpr (FMT == CUTB_Q4_0) {
    const uint32_t pa = rowA + 36 * t, pb = rowB + 36 * t;
    uint32_t la[9], lb[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) {
      la[k] = lds_u32(pa + 4 * k);
      lb[k] = lds_u32(pb + 4 * k);
    }
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      uint32_t wa[4], wb[4];
      float dA, dB;
      if (pass == 0) {
        wa[0] = la[1]; wa[1] = la[2]; wa[2] = la[3]; wa[3] = __byte_perm(la[0], la[4], 0x5432);
        wb[0] = lb[1]; wb[1] = lb[2]; wb[2] = lb[3]; wb[3] = __byte_perm(lb[0], lb[4], 0x5432);
        dA = h2f_bits(la[0] & 0xFFFFu); dB = h2f_bits(lb[0] & 0xFFFFu);
      } else {
        wa[0] = la[5]; wa[1] = la[6]; wa[2] = la[7]; wa[3] = la[8];
        wb[0] = lb[5]; wb[1] = lb[6]; wb[2] = lb[7]; wb[3] = lb[8];
        dA = h2f_bits(la[4] >> 16); dB = h2f_bits(lb[4] >> 16);
      }
      uint32_t al[4], ah[4], bl[4], bh[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        al[i] = nib_lo_s(wa[i]); ah[i] = nib_hi_s(wa[i]);
        bl[i] = nib_lo_s(wb[i]); bh[i] = nib_hi_s(wb[i]);
      }
#pragma unroll
      for (int nt = 0; nt < NVR; ++nt) {
        int c[4], c2[4];
        block_mmas<true>(c, c2, al, bl, ah, bh, actp[nt] + pass * pass_a);
        finish(nt, c, c2, dA, dB, pass * pass_e);
      }
    }
  } else if constexpr (FMT == CUTB_Q8_0) {
    const uint32_t pa = rowA + 68 * t, pb = rowB + 68 * t;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      uint32_t wa[8], wb[8];
      float dA, dB;
      if (pass == 0) {
        const uint32_t a0 = lds_u32(pa), b0 = lds_u32(pb), a8 = lds_u32(pa + 32), b8 = lds_u32(pb + 32);
#pragma unroll
        for (int k = 0; k < 7; ++k) {
          wa[k] = lds_u32(pa + 4 + 4 * k);
          wb[k] = lds_u32(pb + 4 + 4 * k);
        }
        wa[7] = __byte_perm(a0, a8, 0x5432);
        wb[7] = __byte_perm(b0, b8, 0x5432);
        dA = h2f_bits(a0 & 0xFFFFu); dB = h2f_bits(b0 & 0xFFFFu);
      } else {
        dA = h2f_bits(lds_u32(pa + 32) >> 16); dB = h2f_bits(lds_u32(pb + 32) >> 16);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          wa[k] = lds_u32(pa + 36 + 4 * k);
          wb[k] = lds_u32(pb + 36 + 4 * k);
        }
      }
#pragma unroll
      for (int nt = 0; nt < NVR; ++nt) {
        const uint32_t r0a[4] = {wa[0], wa[2], wa[4], wa[6]}, r1a[4] = {wa[1], wa[3], wa[5], wa[7]};
        const uint32_t r0b[4] = {wb[0], wb[2], wb[4], wb[6]}, r1b[4] = {wb[1], wb[3], wb[5], wb[7]};
        int c[4], c2[4];
        block_mmas<false>(c, c2, r0a, r0b, r1a, r1b, actp[nt] + pass * pass_a);
        finish(nt, c, c2, dA, dB, pass * pass_e);
      }
    }
  } else {  // Q4_K: lane t owns the 64-weight group t = sub-blocks 2t (low nibbles) and 2t+1 (high nibbles)
    const uint4 hA = lds_u128(rowA), hB = lds_u128(rowB);
    const uint4 qa0 = lds_u128(rowA + 16 + 32 * t), qa1 = lds_u128(rowA + 32 + 32 * t);
    const uint4 qb0 = lds_u128(rowB + 16 + 32 * t), qb1 = lds_u128(rowB + 32 + 32 * t);
    const uint32_t wa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
    const uint32_t wb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
    const float dA = h2f_bits(hA.x & 0xFFFFu), mA = h2f_bits(hA.x >> 16);
    const float dB = h2f_bits(hB.x & 0xFFFFu), mB = h2f_bits(hB.x >> 16);
    // 6-bit (scale, min) fields of this lane's two sub-blocks (gguf_reader.cpp:668-676)
    const bool upper = t >= 2;  // sub-blocks 4..7 keep their high bits elsewhere
    const uint32_t scA = upper ? (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u) : hA.y & 0x3F3F3F3Fu;
    const uint32_t mnA = upper ? ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u) : hA.z & 0x3F3F3F3Fu;
    const uint32_t scB = upper ? (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u) : hB.y & 0x3F3F3F3Fu;
    const uint32_t mnB = upper ? ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u) : hB.z & 0x3F3F3F3Fu;
    const float ndA = -dA * 8388608.f, nmA = -mA * 8388608.f, ndB = -dB * 8388608.f, nmB = -mB * 8388608.f;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const uint32_t sel = 0x7540u | (((2 * t) & 3) + pass);
      // d * (2^23 + sc) - d * 2^23 == d * sc exactly
      const float dsA = fmaf(dA, __uint_as_float(__byte_perm(scA, 0x4B000000u, sel)), ndA);
      const float dmA = fmaf(mA, __uint_as_float(__byte_perm(mnA, 0x4B000000u, sel)), nmA);
      const float dsB = fmaf(dB, __uint_as_float(__byte_perm(scB, 0x4B000000u, sel)), ndB);
      const float dmB = fmaf(mB, __uint_as_float(__byte_perm(mnB, 0x4B000000u, sel)), nmB);
      uint32_t fa[8], fb[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        fa[k] = (pass ? (wa[k] >> 4) : wa[k]) & 0x0F0F0F0Fu;
        fb[k] = (pass ? (wb[k] >> 4) : wb[k]) & 0x0F0F0F0Fu;
      }
#pragma unroll
      for (int nt = 0; nt < NVR; ++nt) {
        const uint32_t r0a[4] = {fa[0], fa[2], fa[4], fa[6]}, r1a[4] = {fa[1], fa[3], fa[5], fa[7]};
        const uint32_t r0b[4] = {fb[0], fb[2], fb[4], fb[6]}, r1b[4] = {fb[1], fb[3], fb[5], fb[7]};
        int c[4], c2[4];
        block_mmas<true>(c, c2, r0a, r0b, r1a, r1b, actp[nt] + pass * pass_a);
        finish(nt, c, c2, dsA, dsB, pass * pass_e);
        const float sxv = __uint_as_float(lds_u32(sxp[nt] + pass * pass_e));
        tot[nt][0] = fmaf(-dmA, sxv, tot[nt][0]);
        tot[nt][1] = fmaf(-dmB, sxv, tot[nt][1]);
      }
    }
  }
}

// One stage of one warp: 16 rows x ngr granules of raw blocks at shared
// address `st`.  `actb` / `escb` / `sxb` point at the staged activations,
// scales and (Q4_K) scaled sums of the first 32-k block of the stage.
template <int FMT, int NT, int PS>
__device__ __forceinline__ void compute_stage(uint32_t st, uint32_t ngr, uint32_t actb, uint32_t act_stride,
                                              const uint32_t (&aoff)[NT], uint32_t escb, uint32_t sxb, uint32_t g,
                                              uint32_t t, float (&tot)[NT][2]) {
  constexpr uint32_t NV = NT * 4;
  const uint32_t rowA = st + g * PS, rowB = rowA + gv_raw_row(FMT);  // tile rows 2g and 2g + 1

  // scale the exact integer block dot products and accumulate in fp32
  auto accumulate = [&](uint32_t kb, float dA, float dB, const uint32_t (&fa)[2], const uint32_t (&fb)[2]) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint2 x = lds_u64(actb + kb * act_stride + aoff[nt]);
      const float e = __uint_as_float(lds_u32(escb + (kb * NV + nt * 4 + t) * 4));
      int c[4];
      mma_i8<FMT == CUTB_Q4_0>(c, fa[0], fb[0], fa[1], fb[1], x.x, x.y);
      const float fg = (float)(c[0] * 256 + c[1]), fh = (float)(c[2] * 256 + c[3]);
      if constexpr (FMT == CUTB_Q4_0) {
        const float off = __uint_as_float(lds_u32(sxb + (kb * NV + nt * 4 + t) * 4));
        tot[nt][0] = fmaf(dA, fmaf(e, fg, -off), tot[nt][0]);
        tot[nt][1] = fmaf(dB, fmaf(e, fh, -off), tot[nt][1]);
      } else {
        tot[nt][0] = fmaf(dA * e, fg, tot[nt][0]);
        tot[nt][1] = fmaf(dB * e, fh, tot[nt][1]);
      }
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
            mma_i8<true>(c, a0, a1, a2, a3, x.x, x.y);
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

// Balanced int8 digits of |v| <= 32639: v = 256 * hi + lo, both in [-128, 127].  Eight values
// packed four to a word: the low digit is the value's low byte as it stands (read as int8),
// the high digit is byte 1 of value + 128.
__device__ __forceinline__ void pack_digits(const int (&v)[8], uint32_t (&hi)[2], uint32_t (&lo)[2]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t a = (uint32_t)v[4 * h], b = (uint32_t)v[4 * h + 1], c = (uint32_t)v[4 * h + 2], d = (uint32_t)v[4 * h + 3];
    lo[h] = __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
    hi[h] = __byte_perm(__byte_perm(a + 128u, b + 128u, 0x0051), __byte_perm(c + 128u, d + 128u, 0x0051), 0x5410);
  }
}

constexpr float GV_QMAX = 32512.f;

// Stages the activations of blocks [0, nblk) of this K split (starting at k0)
// as two-digit block floating point in MMA fragment order.
//   act  : [blk][col][lane t][8 bytes]; col = 2 * vrow + digit (0 = high digit)
//   esc  : [blk][NV] fp32 scale of the integer dot product (includes the 1/16 of the Q4_0 nibble encoding)
//   sx   : [blk][NV] fp32 e * sum(x^) (Q4_K), 8 e * sum(x^) (Q4_0: the q - 8 offset)
//
// Diagonal variant (DIAG): act is [blk][vrow][digit][MMA i][8 bytes] followed by
// 32 zero bytes, esc / sx are [blk][NT] (NT = number of virtual rows).
template <int FMT, int AMODE, int NT, bool DIAG, int THREADS>
__device__ __forceinline__ void stage_activations(const GvParams &p, uint8_t *act, float *esc, float *sx, uint32_t k0,
                                                  uint32_t nblk, uint32_t ncp, uint32_t tid, const float *nscale) {
  constexpr uint32_t NV = DIAG ? NT : NT * 4;
  const uint32_t nrows = p.M;
  constexpr bool AF32 = AMODE != GV_A_HALF;      // fp32 loads
  constexpr bool TWO = AMODE == GV_A_F32_TWO;     // two 16-bit levels per fp32 value
  const uint32_t nvr = TWO ? 2 * nrows : nrows;
  const uint32_t nchunks = nblk * nrows * 4;
  // rows whose element pairs can be read with one load each (the pair's first element is even)
  const bool pairs = (reinterpret_cast<uintptr_t>(p.A) % (AF32 ? 8 : 4) == 0) && (p.lda % 2 == 0);
  const float wscale = (FMT == CUTB_Q4_0) ? 0.0625f : 1.0f;  // Q4_0 nibbles enter the MMA as 16 q
  const float sxscale = (FMT == CUTB_Q4_0) ? 8.0f : 1.0f;    // Q4_0: the -8 offset of every weight
  for (uint32_t base = 0; base < nchunks; base += THREADS) {  // uniform trip count: shuffles inside
    const uint32_t id = base + tid;
    const bool live = id < nchunks;
    const uint32_t ct = id & 3, q = id >> 2;
    // (a single activation row is the common decode case: no division on its path)
    const uint32_t m = (live && nrows > 1) ? q % nrows : 0, kb = live ? (nrows > 1 ? q / nrows : q) : 0;
    const bool even = (FMT == CUTB_Q4_K) || ((kb & 1) == 0);
    float x[8];
    float amax = 0.f;
    const uint64_t rowbase = (uint64_t)m * p.lda + k0 + kb * 32;
    const float rs = (nscale && live) ? nscale[m] : 1.f;
    // the eight elements of a chunk are four pairs (el, el + 1) with el even: one load per pair when
    // the row is aligned for it.  All loads of a chunk are issued before any is used (idle threads
    // read the row's first elements and discard them).
    const uint64_t rb = live ? rowbase : 0;
    if (pairs) {
      if constexpr (AF32) {
        float2 v[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
          const uint32_t el = DIAG ? diag_elem<FMT>(even, ct, 2 * i) : frag_elem<FMT>(even, ct, 2 * i);
          v[i] = __ldg(reinterpret_cast<const float2 *>(reinterpret_cast<const float *>(p.A) + rb + el));
        }
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) x[2 * i] = v[i].x, x[2 * i + 1] = v[i].y;
      } else {
        __half2 v[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
          const uint32_t el = DIAG ? diag_elem<FMT>(even, ct, 2 * i) : frag_elem<FMT>(even, ct, 2 * i);
          v[i] = __ldg(reinterpret_cast<const __half2 *>(reinterpret_cast<const __half *>(p.A) + rb + el));
        }
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
          const float2 f = __half22float2(v[i]);
          x[2 * i] = f.x, x[2 * i + 1] = f.y;
        }
      }
    } else {
#pragma unroll
      for (uint32_t i = 0; i < 8; ++i) {
        const uint32_t el = DIAG ? diag_elem<FMT>(even, ct, i) : frag_elem<FMT>(even, ct, i);
        x[i] = load_act<AF32>(p.A, rb + el);
      }
    }
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
      if (!live) x[i] = 0.f;
      if (nscale && live) {  // RMSNorm fused into the staging
        const uint32_t el = DIAG ? diag_elem<FMT>(even, ct, i) : frag_elem<FMT>(even, ct, i);
        x[i] = x[i] * rs * __ldg(p.norm_w + k0 + kb * 32 + el);
      }
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
    uint32_t whi[2], wlo[2];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = __float2int_rn(x[i] * inv);
      isum += v[i];
    }
    pack_digits(v, whi, wlo);
    const uint32_t vr = TWO ? 2 * m : m;
    if constexpr (FMT != CUTB_Q8_0) {
      isum += __shfl_xor_sync(0xffffffffu, isum, 1);
      isum += __shfl_xor_sync(0xffffffffu, isum, 2);
    }
    // byte offset of (block, virtual row, digit, chunk) in the staged layout
    auto act_off = [&](uint32_t vrow, uint32_t digit) -> size_t {
      if constexpr (DIAG) return (((size_t)kb * NT + vrow) * 2 + digit) * 32 + ct * 8;
      return ((size_t)(kb * ncp + 2 * vrow + digit) * 4 + ct) * 8;
    };
    if (live) {
      *reinterpret_cast<uint2 *>(act + act_off(vr, 0)) = make_uint2(whi[0], whi[1]);
      *reinterpret_cast<uint2 *>(act + act_off(vr, 1)) = make_uint2(wlo[0], wlo[1]);
      if (ct == 0) {
        esc[kb * NV + vr] = e * wscale;
        if constexpr (FMT != CUTB_Q8_0) sx[kb * NV + vr] = sxscale * e * (float)isum;
      }
    }
    if constexpr (TWO) {
      // second 16-bit level: the residual x - x^ e, at scale e / 65024
      const float e2 = e * (1.0f / (2.f * GV_QMAX)), inv2 = inv * (2.f * GV_QMAX);
      int w[8], isum2 = 0;
      uint32_t rhi[2], rlo[2];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float r = fmaf(-(float)v[i], e, x[i]);
        w[i] = __float2int_rn(r * inv2);
        isum2 += w[i];
      }
      pack_digits(w, rhi, rlo);
      if constexpr (FMT != CUTB_Q8_0) {
        isum2 += __shfl_xor_sync(0xffffffffu, isum2, 1);
        isum2 += __shfl_xor_sync(0xffffffffu, isum2, 2);
      }
      if (live) {
        *reinterpret_cast<uint2 *>(act + act_off(vr + 1, 0)) = make_uint2(rhi[0], rhi[1]);
        *reinterpret_cast<uint2 *>(act + act_off(vr + 1, 1)) = make_uint2(rlo[0], rlo[1]);
        if (ct == 0) {
          esc[kb * NV + vr + 1] = e2 * wscale;
          if constexpr (FMT != CUTB_Q8_0) sx[kb * NV + vr + 1] = sxscale * e2 * (float)isum2;
        }
      }
    }
  }
  if constexpr (DIAG) {
    // lanes whose MMA columns belong to another lane's block read these zeros
    if (tid < 8) reinterpret_cast<uint32_t *>(act + (size_t)p.gran_per_split * 8 * NT * 64)[tid] = 0u;
    return;
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
      if constexpr (FMT != CUTB_Q8_0) sx[o] = 0.f;
    }
}

// 1 / rms of every activation row (fused RMSNorm), by GV_WARPS * 32 threads synchronising on named
// barrier 1: red[GV_WARPS * 16 + m] holds row m's scale on return.  `red` needs GV_WARPS * 16 + 16 floats.
template <bool AF32N>
__device__ __forceinline__ void rms_scales(const GvParams &p, float *red, uint32_t tid) {
  const uint32_t warp = tid >> 5, lane = tid & 31;
  for (uint32_t m = 0; m < p.M; ++m) {
    float ss = 0.f;
    // K is a multiple of 256: two elements per thread and pass, four passes' loads in flight
    for (uint32_t k = 2 * tid; k < p.K; k += 8 * GV_WARPS * 32) {
      float v[8];
#pragma unroll
      for (uint32_t u = 0; u < 4; ++u) {
        const uint32_t kk = k + u * 2 * GV_WARPS * 32;
        const bool in = kk < p.K;
        v[2 * u] = in ? load_act<AF32N>(p.A, (uint64_t)m * p.lda + kk) : 0.f;
        v[2 * u + 1] = in ? load_act<AF32N>(p.A, (uint64_t)m * p.lda + kk + 1) : 0.f;
      }
#pragma unroll
      for (uint32_t u = 0; u < 8; ++u) ss = fmaf(v[u], v[u], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp * 16 + m] = ss;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");
  if (tid < p.M) {
    float ss = 0.f;
#pragma unroll
    for (int w = 0; w < GV_WARPS; ++w) ss += red[w * 16 + tid];
    red[GV_WARPS * 16 + tid] = rsqrtf(ss / (float)p.K + p.norm_eps);
  }
  asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");
}

// Stages the activations of one launch once, for all its CTAs: block (x, y) stages a run of 32-k blocks
// of K split y into that split's blob, in exactly the layout (and with exactly the arithmetic) a mat-vec
// CTA would build in its own shared memory.  Used from three virtual rows up, where every CTA repeating
// the staging costs more than the mat-vec itself.
template <int FMT, int AMODE, int NT>
__global__ void __launch_bounds__(GV_WARPS * 32) stage_acts_kernel(const GvParams p, uint32_t ncp, uint32_t blocks_per_cta) {
  __shared__ float red[GV_WARPS * 16 + 16];
  constexpr uint32_t NV = NT * 4;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations may come from the kernel before
  const uint32_t tid = threadIdx.x;
  const uint32_t G = p.K >> 8;
  const uint32_t gs0 = blockIdx.y * p.gran_per_split;
  const uint32_t gs1 = min(G, gs0 + p.gran_per_split);
  const uint32_t nblk = (gs1 - gs0) * 8, nblk_alloc = p.gran_per_split * 8;
  const uint32_t b0 = blockIdx.x * blocks_per_cta;  // even: block parity decides the fragment order
  const float *nscale = nullptr;
  if (p.norm_w) {
    rms_scales<AMODE != GV_A_HALF>(p, red, tid);
    nscale = red + GV_WARPS * 16;
  }
  if (b0 >= nblk) return;
  const uint32_t nb = min(blocks_per_cta, nblk - b0);
  uint8_t *base = p.staged + (size_t)blockIdx.y * p.staged_bytes;
  float *esc0 = reinterpret_cast<float *>(base + (size_t)nblk_alloc * ncp * 32);
  float *sx0 = esc0 + (size_t)nblk_alloc * NV;
  stage_activations<FMT, AMODE, NT, false, GV_WARPS * 32>(p, base + (size_t)b0 * ncp * 32, esc0 + (size_t)b0 * NV, sx0 + (size_t)b0 * NV,
                                                          gs0 * 256 + b0 * 32, nb, ncp, tid, nscale);
}

// MINB: CTAs per SM the register budget is kept under -- 2 where this launch's CTA and the next launch's share an
// SM, 1 for the plans whose shared memory fills the SM anyway (then up to 120 registers instead of 56).
template <int FMT, int AMODE, int NT, bool DIAG, int MINB>
__global__ void __launch_bounds__(GV_THREADS, MINB) qgemv_blocks_kernel(const GvParams p) {
  constexpr int PS = gv_pair_stride(FMT, DIAG);
  constexpr uint32_t RAWROW = gv_raw_row(FMT);
  constexpr uint32_t GB = granule_bytes(FMT);
  constexpr uint32_t STAGE_BYTES = (GV_ROWS / 2) * PS;
  constexpr uint32_t NV = DIAG ? NT : NT * 4, NC8 = NT * 8;
  extern __shared__ __align__(128) uint8_t smem[];

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  constexpr bool TWO = AMODE == GV_A_F32_TWO;
  const uint32_t nvr = TWO ? 2 * p.M : p.M;  // virtual activation rows (two per fp32 row staged at two levels)
  const uint32_t ncols = 2 * nvr;
  const uint32_t ncp = (ncols < NC8) ? ncols + 1 : ncols;
  const uint32_t nblk_alloc = p.gran_per_split * 8;
  const uint32_t S = p.stages;

  uint8_t *ring = smem;
  uint8_t *act = ring + (size_t)S * STAGE_BYTES;
  float *esc = reinterpret_cast<float *>(act + (DIAG ? (size_t)nblk_alloc * NT * 64 + 32 : (size_t)nblk_alloc * ncp * 32));
  float *sx = esc + nblk_alloc * NV;
  float *red = sx + (FMT != CUTB_Q8_0 ? nblk_alloc * NV : 0);  // two buffers of [GV_WARPS][16][NV]
  uint64_t *bars = reinterpret_cast<uint64_t *>(red + 2 * GV_WARPS * GV_ROWS * NV);  // full[S], empty[S]

  // rows of this CTA and granules (256 weights) of this K split; a stage holds
  // 16 rows x up to GV_KC granules, one granule per consumer warp
  const uint32_t unit = p.glu ? 2u : 1u;  // paired rows stay in one CTA (and, ranges being even, in one tile)
  const uint32_t r0 = (uint32_t)((uint64_t)blockIdx.x * (p.N / unit) / gridDim.x) * unit;
  const uint32_t r1 = (uint32_t)((uint64_t)(blockIdx.x + 1) * (p.N / unit) / gridDim.x) * unit;
  const uint32_t G = p.K >> 8;
  const uint32_t gs0 = blockIdx.y * p.gran_per_split;
  const uint32_t gs1 = min(G, gs0 + p.gran_per_split);
  const uint32_t ng = gs1 - gs0;
  const uint32_t cpt = (ng + GV_KC - 1) / GV_KC;  // K chunks (stages) per row tile
  const uint32_t ntiles = (r1 - r0 + GV_ROWS - 1) / GV_ROWS;
  const uint32_t total_stages = ntiles * cpt;

  const uint32_t ring_u = smem_u32(ring);
  // Q8_0: two barrier pairs per ring slot.  The K halves of a stage (8 granules, 8 warps each)
  // are copied, consumed and handed back independently, which halves the copy-issue time
  // inside the release -> refill -> consume loop of a slot.  The 4-bit formats keep whole
  // rows per copy: their half rows (1152 bytes) cost more in copy efficiency than the
  // shorter loop wins.
  constexpr uint32_t HV = FMT == CUTB_Q8_0 ? 2u : 1u;
  const uint32_t full_u = smem_u32(bars), empty_u = full_u + S * HV * 8;

  // Let the next kernel of the stream start its own prologue and weight
  // prefetch as soon as an SM has room for it (programmatic dependent launch).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (tid == 0) {
    for (uint32_t s = 0; s < HV * S; ++s) {
      mbar_init(full_u + s * 8, 1);
      mbar_init(empty_u + s * 8, GV_WARPS / HV);
    }
    mbar_init(full_u + 4 * S * 8, 1);  // arrival of the pre-staged activations
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == GV_WARPS) {
    // ---- producer warp: whole row segments, one bulk copy per row and stage ----
    bool dead = false;
    uint32_t tile = 0, c = 0, slot = 0, par = 1u;  // par: parity of the slot's previous use
    for (uint32_t j = 0; j < total_stages && !dead; ++j) {
      const uint32_t row_base = r0 + tile * GV_ROWS;
      const uint32_t valid = min((uint32_t)GV_ROWS, r1 - row_base);
      for (uint32_t h = 0; h < HV && !dead; ++h) {
        if (j >= S) {
          const bool ok = mbar_wait_probe_first(empty_u + (slot * HV + h) * 8, par);
          if (!__all_sync(0xffffffffu, ok)) {
            dead = true;
            if (lane == 0 && p.status) atomicExch(p.status, (int)CUTB_ERR_TIMEOUT);
            break;
          }
        }
        const uint32_t gq = gs0 + c * GV_KC + h * (GV_KC / HV);
        const uint32_t bytes = gq < gs1 ? min((uint32_t)(GV_KC / HV), gs1 - gq) * GB : 0u;
        const uint32_t bar = full_u + (slot * HV + h) * 8;
        if (lane == 0) mbar_arrive_expect_tx(bar, valid * bytes);  // zero bytes: the phase completes at once
        __syncwarp();
        if (HV == 1 && bytes == RAWROW && p.row_bytes == RAWROW) {
          // the stage holds whole rows: tile rows 2i and 2i + 1 are one contiguous range, one copy per pair
          if (2 * lane < valid)
            bulk_g2s(ring_u + slot * STAGE_BYTES + lane * PS, p.W + (uint64_t)(row_base + 2 * lane) * p.row_bytes,
                     (2 * lane + 1 < valid) ? 2 * RAWROW : RAWROW, bar);
        } else if (bytes && lane < valid) {
          bulk_g2s(ring_u + slot * STAGE_BYTES + (lane >> 1) * PS + (lane & 1) * RAWROW + h * (GV_KC / HV) * GB,
                   p.W + (uint64_t)(row_base + lane) * p.row_bytes + (uint64_t)gq * GB, bytes, bar);
        }
      }
      if (++slot == S) slot = 0, par ^= 1u;
      if (++c == cpt) c = 0, ++tile;
    }
    // stay resident until every copy issued here has landed (bounded)
    const uint32_t first = total_stages > S ? total_stages - S : 0;
    for (uint32_t j = first; j < total_stages; ++j)
      for (uint32_t h = 0; h < HV; ++h) (void)mbar_wait_bounded(full_u + ((j % S) * HV + h) * 8, (j / S) & 1u);
    return;
  }

  // ---- consumer warps ---------------------------------------------------------
  // Everything above only read the (constant) weights.  The activations, D and
  // C may belong to the previous kernel of the stream: wait for it to finish.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  bool dead = false;
  bool fetched = false;
  if constexpr (!DIAG) fetched = p.staged != nullptr;
  if (fetched) {
    // the launch before this one staged the activations of every K split once; fetch this split's
    // (the same bytes this CTA would have produced) with bulk copies
    const uint32_t abar = full_u + 4 * S * 8;
    if (warp == 0) {
      if (lane == 0) mbar_arrive_expect_tx(abar, p.staged_bytes);
      __syncwarp();
      const uint8_t *src = p.staged + (size_t)blockIdx.y * p.staged_bytes;
      for (uint32_t off = lane * 8192u; off < p.staged_bytes; off += 32u * 8192u)
        bulk_g2s(smem_u32(act) + off, src + off, min(8192u, p.staged_bytes - off), abar);
    }
    const bool ok = mbar_wait_probe_first(abar, 0);
    if (!__all_sync(0xffffffffu, ok)) {
      dead = true;
      if (lane == 0 && p.status) atomicExch(p.status, (int)CUTB_ERR_TIMEOUT);
    }
  } else {
    const float *nscale = nullptr;
    if (p.norm_w) {
      // fused RMSNorm: every CTA needs the scale of the whole row, whatever K slice it stages; the
      // reduction buffers are idle until the first tile
      rms_scales<AMODE != GV_A_HALF>(p, red, tid);
      nscale = red + GV_WARPS * 16;
    }
    stage_activations<FMT, AMODE, NT, DIAG, GV_WARPS * 32>(p, act, esc, sx, gs0 * 256, ng * 8, ncp, tid, nscale);
  }
  asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");

  const uint32_t act_u = smem_u32(act), act_stride = ncp * 32, esc_u = smem_u32(esc), sx_u = smem_u32(sx);
  // per-lane activation fragment offsets (idle lanes read zeros)
  uint32_t aoff[NT];
  // diagonal variant: MMA column g belongs to the block pair of lane g >> 1, digit g & 1
  const bool mine = (t == (g >> 1));
  const uint32_t zero_u = act_u + nblk_alloc * NT * 64;
  const uint32_t pass_a = mine ? NT * 64u : 0u, gran_a = mine ? 8u * NT * 64u : 0u;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    if constexpr (DIAG) {
      aoff[nt] = mine ? (((2 * t) * NT + nt) * 2 + (g & 1)) * 32 : 0u;
    } else {
      const uint32_t col = nt * 8 + g;
      aoff[nt] = ((col < ncols ? col : ncols) * 4 + t) * 8;
    }
  }

  uint32_t slot = 0, parity = 0;
  const uint32_t hv = HV == 2 ? warp >> 3 : 0u;  // the K half this warp's granule belongs to
  for (uint32_t tile = 0; tile < ntiles; ++tile) {
    float tot[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = 0.f;

    for (uint32_t c = 0; c < cpt; ++c) {
      if (!dead && !mbar_test(full_u + (slot * HV + hv) * 8, parity)) {  // the vote only on the slow path
        const bool ok = mbar_wait_bounded(full_u + (slot * HV + hv) * 8, parity);
        if (!__all_sync(0xffffffffu, ok)) {
          dead = true;
          if (lane == 0 && p.status) atomicExch(p.status, (int)CUTB_ERR_TIMEOUT);
        }
      }
      const uint32_t gq = gs0 + c * GV_KC + warp;  // this warp's granule of the chunk
      if (!dead && gq < gs1) {
        const uint32_t kb0 = (gq - gs0) * 8;  // first 32-weight block of the granule inside the split
        if constexpr (DIAG) {
          uint32_t actp[NT], escp[NT], sxp[NT];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            actp[nt] = mine ? act_u + (gq - gs0) * gran_a + aoff[nt] : zero_u;
            escp[nt] = esc_u + ((kb0 + 2 * t) * NT + nt) * 4;
            sxp[nt] = sx_u + ((kb0 + 2 * t) * NT + nt) * 4;
          }
          compute_granule_diag<FMT, NT>(ring_u + slot * STAGE_BYTES + warp * GB + g * PS, actp, pass_a, escp, sxp,
                                            NT * 4, t, tot);
        } else {
          compute_stage<FMT, NT, PS>(ring_u + slot * STAGE_BYTES + warp * GB, 1, act_u + kb0 * act_stride, act_stride,
                                     aoff, esc_u + kb0 * NV * 4, sx_u + kb0 * NV * 4, g, t, tot);
        }
      }
      __syncwarp();
      asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, %1, 0;\n\t@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" ::"r"(
                       empty_u + (slot * HV + hv) * 8),
                   "r"(lane)
                   : "memory");
      if (++slot == S) slot = 0, parity ^= 1u;
    }

    // meet the other warps' K slices in a fixed order (double-buffered: one barrier per tile)
    float *rbuf = red + (size_t)(tile & 1) * GV_WARPS * GV_ROWS * NV;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if constexpr (DIAG) {
        // the four lanes of a quad hold partial sums of the same virtual row
        float a = tot[nt][0], b = tot[nt][1];
        a += __shfl_xor_sync(0xffffffffu, a, 1);
        b += __shfl_xor_sync(0xffffffffu, b, 1);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        b += __shfl_xor_sync(0xffffffffu, b, 2);
        if (t == 0) {
          float *r = rbuf + ((size_t)warp * GV_ROWS) * NV + nt;
          r[(2 * g) * NV] = a;      // MMA row g = tile row 2g
          r[(2 * g + 1) * NV] = b;  // MMA row g + 8 = tile row 2g + 1
        }
      } else {
        float *r = rbuf + ((size_t)warp * GV_ROWS) * NV + nt * 4 + t;
        r[(2 * g) * NV] = tot[nt][0];
        r[(2 * g + 1) * NV] = tot[nt][1];
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");
    const uint32_t row_base = r0 + tile * GV_ROWS;
    auto row_sum = [&](uint32_t row, uint32_t m) -> float {
      float sum = 0.f;
      if constexpr (TWO) {
#pragma unroll
        for (int w = 0; w < GV_WARPS; ++w) {
          const float2 hl = *reinterpret_cast<const float2 *>(rbuf + ((size_t)w * GV_ROWS + row) * NV + 2 * m);
          sum += hl.x + hl.y;
        }
      } else {
#pragma unroll
        for (int w = 0; w < GV_WARPS; ++w) sum += rbuf[((size_t)w * GV_ROWS + row) * NV + m];
      }
      return sum;
    };
    if (p.glu) {  // (gate, up) row pairs: one output per pair
      for (uint32_t o = tid; o < (GV_ROWS / 2) * p.M; o += GV_WARPS * 32) {
        const uint32_t pr = o % (GV_ROWS / 2), m = o / (GV_ROWS / 2), n = row_base + 2 * pr;
        if (n < r1)
          p.C[(size_t)m * p.ldc + (n >> 1)] = apply_epilogue(row_sum(2 * pr, m), CUTB_FUSION_UNARY, p.fusion_op, 0.f) * row_sum(2 * pr + 1, m);
      }
      continue;
    }
    for (uint32_t o = tid; o < GV_ROWS * p.M; o += GV_WARPS * 32) {
      const uint32_t row = o % GV_ROWS, m = o / GV_ROWS, n = row_base + row;
      if (n < r1) {
        const float sum = row_sum(row, m);
        if (p.ksplit > 1) {
          p.partial[((size_t)blockIdx.y * p.M + m) * p.N + n] = sum;
        } else {
          const float dv = (p.fusion_type == CUTB_FUSION_BINARY) ? p.D[(size_t)m * p.ldd + n] : 0.f;
          const float out = apply_epilogue(sum, p.fusion_type, p.fusion_op, dv);
          if (p.world > 1) {
            const size_t at = (size_t)m * p.ldc_total + p.n_off + n;
            for (uint32_t q = 0; q < p.world; ++q) p.peer_C[q][at] = out;
          } else {
            p.C[(size_t)m * p.ldc + n] = out;
          }
        }
      }
    }
  }
}

// Destination of a row-sharded scatter (world > 1) as the kernels see it.
struct ScatterArgs {
  uint32_t world, n_off, ldc_total;
  float *peer_C[CUTB_MAX_PEERS];
};

// Fixed-order sum of the K-split partials followed by the fused epilogue; with a scatter
// destination the result goes to every rank's full output.
__global__ void splitk_reduce_kernel(const float *__restrict__ partial, float *__restrict__ C, const float *__restrict__ D,
                                     uint32_t M, uint32_t N, uint32_t ldc, uint32_t ldd, uint32_t ksplit, int ftype, int fop,
                                     const ScatterArgs sc) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < M * N) {
    const uint32_t m = i / N, n = i % N;
    float sum = 0.f;
    for (uint32_t s = 0; s < ksplit; ++s) sum += partial[((size_t)s * M + m) * N + n];
    const float dv = (ftype == CUTB_FUSION_BINARY) ? D[(size_t)m * ldd + n] : 0.f;
    const float out = apply_epilogue(sum, ftype, fop, dv);
    if (sc.world > 1) {
      const size_t at = (size_t)m * sc.ldc_total + sc.n_off + n;
      for (uint32_t q = 0; q < sc.world; ++q) sc.peer_C[q][at] = out;
    } else {
      C[(size_t)m * ldc + n] = out;
    }
  }
}

// The step boundary of the fused exchange, one small block per rank and step.  Everything the
// earlier kernels of this stream stored into peer memory happened before this kernel (stream
// order); a system-scope fence followed by one system-scope add on every rank's arrival counter
// publishes it.  Then one thread polls this rank's own counter (system-scope acquire loads) until
// all `world` ranks have signalled this step, for at most about a second; on expiry it records
// CUTB_ERR_TIMEOUT and returns, so the stream and the context stay usable.  The step number lives
// on the device (*step_counter), so the same launch can be replayed from a CUDA graph.  Kernels
// after it in the stream see every rank's slice.
struct ExchangeArgs {
  uint32_t world, rank;
  unsigned long long *flag[CUTB_MAX_PEERS];
};
__global__ void peer_exchange_kernel(const ExchangeArgs a, unsigned long long *step_counter, int *status) {
  __shared__ unsigned long long step;
  // Launched with programmatic stream serialization: the mat-vec behind this kernel may start its weight prefetch
  // now (it waits for this kernel's completion before it touches activations or outputs); this kernel itself waits
  // for the kernels before it -- whose peer stores it publishes -- to complete and flush.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) step = ++*step_counter;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world) atomicAdd_system(a.flag[threadIdx.x], 1ull);
  if (threadIdx.x != 0) return;
  const unsigned long long expected = step * a.world;
  const long long t0 = clock64();
  const long long limit = 2000000000ll;  // cycles: about a second at 2 GHz
  for (;;) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(a.flag[a.rank]) : "memory");
    if (v >= expected) return;
    if (clock64() - t0 > limit) {
      if (status) atomicExch(status, (int)CUTB_ERR_TIMEOUT);
      return;
    }
    __nanosleep(100);
  }
}

// ---- host side ---------------------------------------------------------------

int gv_amode(const cutb_qmatmul_desc &d) {
  if (d.a_dtype != CUTB_F32) return GV_A_HALF;
  return (d.flags & CUTB_FLAG_ACT_16BIT) ? GV_A_F32_ONE : GV_A_F32_TWO;
}

struct GvPlan {
  uint32_t nt, nvr, ncp, grid_x, ksplit, gran_per_split, stages;
  bool diag, overlap, pair;
  size_t smem;
  // activations staged once per launch by stage_acts_kernel (otherwise by every CTA)
  bool prestage;
  uint32_t staged_bytes;    // one K split's blob
  uint64_t partial_bytes;   // split-K partial sums, rounded up to 256: the blobs follow them in the workspace
};

size_t gv_smem_bytes(int fmt, bool diag, uint32_t stages, uint32_t nt, uint32_t ncp, uint32_t gran_per_split) {
  const size_t nblk = (size_t)gran_per_split * 8;
  const size_t nv = diag ? nt : nt * 4;
  size_t b = (size_t)stages * (GV_ROWS / 2) * gv_pair_stride(fmt, diag);
  b += diag ? nblk * nt * 64 + 32 : nblk * ncp * 32;
  b += nblk * nv * 4 * (fmt != CUTB_Q8_0 ? 2 : 1);
  b += (size_t)2 * GV_WARPS * GV_ROWS * nv * 4;
  b += 4 * stages * 8 + 8;  // full / empty barriers of both K halves of every slot; arrival of pre-staged activations
  return b;
}

bool gv_plan(const cutb_qmatmul_desc &d, const DeviceInfo &di, GvPlan *pl) {
  const bool af32 = gv_amode(d) == GV_A_F32_TWO;  // two virtual rows per activation row
  pl->nvr = af32 ? 2 * d.M : d.M;
  if (pl->nvr == 0 || pl->nvr > 16) return false;
  // one virtual row: the diagonal variant (nt = virtual rows); otherwise 4 virtual rows per MMA n-tile
  // measured: with two virtual rows the diagonal variant only pays for two fp16 rows of Q8_0
  // (elsewhere its second row costs registers and spills: Q4_K 13.4 -> 10.5 us, fp32 rows 10 % faster shared-k)
  pl->diag = pl->nvr == 1 || (pl->nvr == 2 && !af32 && d.format == CUTB_Q8_0);
  pl->nt = pl->diag ? pl->nvr : (pl->nvr <= 4 ? 1 : (pl->nvr <= 8 ? 2 : 4));
  const uint32_t ncols = 2 * pl->nvr;
  pl->ncp = ncols < pl->nt * 8 ? ncols + 1 : ncols;
  const uint32_t G = d.K / 256;
  const uint32_t tiles = (d.N + GV_ROWS - 1) / GV_ROWS;
  pl->grid_x = tiles < (uint32_t)di.sm_count ? tiles : (uint32_t)di.sm_count;
  uint32_t want = 1;
  if (pl->grid_x * 2 <= (uint32_t)di.sm_count) want = (uint32_t)di.sm_count / pl->grid_x;
  if (want > G) want = G;
  const size_t limit = di.smem_optin;
  // Two CTAs per SM (this launch's and the next one's, which prefetches while
  // this one computes) need <= half of the SM's shared memory each; when that
  // cannot hold two stages, take the deepest ring that fits one CTA per SM.
  // K is split further only when even two stages do not fit.
  const size_t half = (di.smem_per_sm > 2048 ? di.smem_per_sm / 2 - 1024 : limit / 2);
  uint32_t max_stages = 4;
  if (const char *e = getenv("CUTB_GV_STAGES")) max_stages = (uint32_t)atoi(e) < 2 ? 2u : (uint32_t)atoi(e);  // tuning override
  for (uint32_t ks = want; ks <= G; ++ks) {
    const uint32_t gps = (G + ks - 1) / ks;
    // (whatever this launch's own overlap flag says: a CTA above half an SM keeps the NEXT launch from becoming
    // resident under this one's tail.  Measured on the 32-layer decode step: a four-slot ring for the launches that
    // do not overlap themselves cost 17 % of the step, 540 -> 451 tok/s.)
    const bool pair = gv_smem_bytes(d.format, pl->diag, 2, pl->nt, pl->ncp, gps) <= half;
    for (uint32_t st = pair ? 2 : max_stages; st >= 2; --st) {
      const size_t sm = gv_smem_bytes(d.format, pl->diag, st, pl->nt, pl->ncp, gps);
      if (sm <= limit) {
        pl->gran_per_split = gps;
        pl->ksplit = (G + gps - 1) / gps;
        pl->stages = st;
        pl->smem = sm;
        pl->pair = pair;
        // A split forced by shared memory (many activation rows, long K) must not push the launch into a
        // second wave: CTAs this large sit one to an SM, so give every CTA more rows instead.
        if (!pair && (uint64_t)pl->grid_x * pl->ksplit > (uint32_t)di.sm_count) {
          const uint32_t gx = (uint32_t)di.sm_count / pl->ksplit;
          pl->grid_x = gx ? gx : 1;
        }
        const uint32_t nv = pl->diag ? pl->nt : pl->nt * 4;
        // From three virtual rows up the staging, repeated by every CTA, outweighs the mat-vec (measured:
        // 11008 x 4096 Q4_0, batch 8: 17.6 us, of which about 10 us staging): stage once, in a launch of its own.
        pl->prestage = !pl->diag && pl->nvr >= 3 && !(d.flags & CUTB_FLAG_STAGE_PER_CTA);
        if (const char *e = getenv("CUTB_GV_PRESTAGE")) pl->prestage = pl->prestage && atoi(e) != 0;  // tuning override
        pl->staged_bytes = gps * 8 * (pl->ncp * 32 + nv * 4 * (d.format != CUTB_Q8_0 ? 2 : 1));
        pl->partial_bytes = pl->ksplit > 1 ? ((uint64_t)pl->ksplit * d.M * d.N * sizeof(float) + 255) / 256 * 256 : 0;
        return true;
      }
    }
  }
  return false;
}

uint64_t gv_workspace_need(const GvPlan &pl) {
  return pl.partial_bytes + (pl.prestage ? (uint64_t)pl.ksplit * pl.staged_bytes : 0);
}

template <int FMT, int AMODE, int NT>
int gv_launch_prestage(const GvParams &p, const GvPlan &pl, cudaStream_t stream) {
  // one pass of the staging loop per CTA: 512 threads = 512 chunks of (block, row, lane) = 128 / M blocks, even
  uint32_t per = (GV_WARPS * 32 / 4) / p.M;
  per = per < 2 ? 2 : per & ~1u;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((pl.gran_per_split * 8 + per - 1) / per, pl.ksplit);
  cfg.blockDim = dim3(GV_WARPS * 32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pl.overlap ? 1 : 0;
  CUTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, stage_acts_kernel<FMT, AMODE, NT>, p, pl.ncp, per));
  return CUTB_OK;
}

template <int FMT, int AMODE, int NT, bool DIAG, int MINB>
int gv_launch_inst(const GvParams &p, const GvPlan &pl, cudaStream_t stream) {
  static bool configured[64] = {};  // per device: the attribute is set once on each
  int dev = 0;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    DeviceInfo di;
    if (int rc = get_device_info(&di)) return rc;
    CUTB_CUDA_TRY(cudaFuncSetAttribute(qgemv_blocks_kernel<FMT, AMODE, NT, DIAG, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)di.smem_optin));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  if constexpr (!DIAG) {
    if (pl.prestage)
      if (int rc = gv_launch_prestage<FMT, AMODE, NT>(p, pl, stream)) return rc;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid_x, pl.ksplit);
  cfg.blockDim = dim3(GV_THREADS);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pl.overlap ? 1 : 0;
  CUTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, qgemv_blocks_kernel<FMT, AMODE, NT, DIAG, MINB>, p));
  return CUTB_OK;
}

template <int FMT, int AMODE>
int gv_launch_nt(const GvParams &p, const GvPlan &pl, cudaStream_t stream) {
  if (pl.diag) return pl.nt == 1 ? gv_launch_inst<FMT, AMODE, 1, true, 2>(p, pl, stream) : gv_launch_inst<FMT, AMODE, 2, true, 2>(p, pl, stream);
  // measured: the 56-register build is the faster one for 4 and 8 virtual rows even where shared memory leaves room
  // for one CTA only (11008 x 4096 Q4_0, batch 8: 12.2 us against 13.7 with 96 registers); 16 rows gain from the
  // larger budget (34.9 -> 28.2 us): no spills, four independent MMA chains per block
  switch (pl.nt) {
    case 1: return gv_launch_inst<FMT, AMODE, 1, false, 2>(p, pl, stream);
    case 2: return gv_launch_inst<FMT, AMODE, 2, false, 2>(p, pl, stream);
    default: return gv_launch_inst<FMT, AMODE, 4, false, 1>(p, pl, stream);  // 16 virtual rows never leave room for a second CTA
  }
}

template <int FMT>
int gv_launch_a(const GvParams &p, const GvPlan &pl, int amode, cudaStream_t stream) {
  switch (amode) {
    case GV_A_HALF: return gv_launch_nt<FMT, GV_A_HALF>(p, pl, stream);
    case GV_A_F32_ONE: return gv_launch_nt<FMT, GV_A_F32_ONE>(p, pl, stream);
    default: return gv_launch_nt<FMT, GV_A_F32_TWO>(p, pl, stream);
  }
}

}  // namespace

bool qgemv_blocks_supported(const cutb_qmatmul_desc &d) {
  if (d.layout != CUTB_LAYOUT_GGUF_BLOCKS) return false;
  if (d.K == 0 || d.K % 256 != 0 || d.N == 0 || d.M == 0) return false;
  const uint32_t nvr = gv_amode(d) == GV_A_F32_TWO ? 2 * d.M : d.M;
  if (nvr > 16) return false;
  if (reinterpret_cast<uintptr_t>(d.W) % 16 != 0) return false;
  return true;
}

// A forced CUTB_VARIANT_GEMV_MMA also takes up to four groups of 16 virtual rows: the weights are streamed once per
// group, which still beats the tensor-core GEMM's fixed cost on narrow weights (a row shard of a projection, a
// 4096-row projection at batch 32).  CUTB_VARIANT_AUTO never picks this; tuning rules do where it measured faster.
uint32_t qgemv_rows_per_group(const cutb_qmatmul_desc &d) { return gv_amode(d) == GV_A_F32_TWO ? 8u : 16u; }

bool qgemv_blocks_supported_in_groups(const cutb_qmatmul_desc &d) {
  if (d.M == 0) return false;
  cutb_qmatmul_desc one = d;
  one.M = d.M < qgemv_rows_per_group(d) ? d.M : qgemv_rows_per_group(d);
  return d.M <= 4 * qgemv_rows_per_group(d) && qgemv_blocks_supported(one) && !(d.flags & CUTB_FLAG_GLU_PAIRS);
}

uint64_t qgemv_blocks_workspace(const cutb_qmatmul_desc &d) {
  const uint32_t per = qgemv_rows_per_group(d);
  if (d.M > per && qgemv_blocks_supported_in_groups(d)) {  // the groups run one after the other on one scratch block
    cutb_qmatmul_desc one = d;
    one.M = per;
    return qgemv_blocks_workspace(one);
  }
  DeviceInfo di;
  if (get_device_info(&di) != CUTB_OK) {
    // no device: report the bound for a 148-SM part so callers can size ahead of time
    di.sm_count = 148;
    di.smem_optin = 232448;
  }
  GvPlan pl;
  if (!qgemv_blocks_supported(d) || !gv_plan(d, di, &pl)) return 0;
  return gv_workspace_need(pl);
}

int qgemv_blocks_launch(const cutb_qmatmul_desc &d, cudaStream_t stream, const cutb_peer_scatter *sc) {
  const uint32_t per = qgemv_rows_per_group(d);
  if (d.M > per && !sc && qgemv_blocks_supported_in_groups(d)) {
    const size_t a_elem = d.a_dtype == CUTB_F32 ? 4 : 2;
    for (uint32_t m0 = 0; m0 < d.M; m0 += per) {
      cutb_qmatmul_desc g = d;
      g.M = d.M - m0 < per ? d.M - m0 : per;
      g.A = reinterpret_cast<const uint8_t *>(d.A) + (size_t)m0 * d.lda * a_elem;
      g.C = d.C + (size_t)m0 * d.ldc;
      if (d.D) g.D = d.D + (size_t)m0 * d.ldd;
      if (int rc = qgemv_blocks_launch(g, stream, nullptr)) return rc;
    }
    return CUTB_OK;
  }
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  GvPlan pl;
  if (!gv_plan(d, di, &pl)) {
    set_last_error("qgemv: no shared-memory plan for M=%u K=%u N=%u", d.M, d.K, d.N);
    return CUTB_ERR_UNSUPPORTED;
  }
  // Flag combinations this kernel cannot run, checked here so that every entry point that reaches the
  // mat-vec (cutb_qmatmul, cutb_qmatmul_scatter, cutb_qmatmul_decode_noalloc) refuses them before a launch.
  if (d.flags & CUTB_FLAG_GLU_PAIRS) {
    if (pl.ksplit > 1 || sc) {
      set_last_error("qgemv: paired gate/up rows need a launch that neither splits K (this shape splits it %u ways) nor scatters to peers",
                     pl.ksplit);
      return CUTB_ERR_UNSUPPORTED;
    }
    if (d.N % 2 != 0) {
      set_last_error("qgemv: paired gate/up rows need an even N, got %u", d.N);
      return CUTB_ERR_INVALID;
    }
  }
  if ((d.flags & CUTB_FLAG_A_RMSNORM) && !d.a_norm_weight) {
    set_last_error("qgemv: CUTB_FLAG_A_RMSNORM without a_norm_weight");
    return CUTB_ERR_INVALID;
  }
  const int amode = gv_amode(d);
  pl.overlap = !(d.flags & CUTB_FLAG_NO_OVERLAP);
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
  p.a_f32 = amode != GV_A_HALF;
  p.norm_w = (d.flags & CUTB_FLAG_A_RMSNORM) ? d.a_norm_weight : nullptr;
  p.norm_eps = d.a_norm_eps;
  p.glu = (d.flags & CUTB_FLAG_GLU_PAIRS) ? 1 : 0;
  p.status = d.status;
  p.world = 0;
  p.n_off = p.ldc_total = 0;
  for (int q = 0; q < CUTB_MAX_PEERS; ++q) p.peer_C[q] = nullptr;
  ScatterArgs sa;
  sa.world = 0;
  sa.n_off = sa.ldc_total = 0;
  for (int q = 0; q < CUTB_MAX_PEERS; ++q) sa.peer_C[q] = nullptr;
  const uint32_t reduce_blocks = (d.M * d.N + 255) / 256;
  if (sc) {
    sa.world = sc->world;
    sa.n_off = sc->n_offset;
    sa.ldc_total = sc->ldc_total;
    for (uint32_t q = 0; q < sc->world; ++q) sa.peer_C[q] = sc->C_peers[q];
    if (pl.ksplit == 1) {  // the mat-vec kernel scatters; with split K its reduction kernel does
      p.world = sa.world;
      p.n_off = sa.n_off;
      p.ldc_total = sa.ldc_total;
      for (uint32_t q = 0; q < sa.world; ++q) p.peer_C[q] = sa.peer_C[q];
    }
  }
  p.staged = nullptr;
  p.staged_bytes = 0;
  if (const uint64_t need = gv_workspace_need(pl)) {
    if (!d.workspace || d.workspace_bytes < need) {
      set_last_error("qgemv: this shape needs %llu workspace bytes (split-K partial sums %llu, staged activations %llu), got %llu",
                     (unsigned long long)need, (unsigned long long)pl.partial_bytes,
                     (unsigned long long)(need - pl.partial_bytes), (unsigned long long)d.workspace_bytes);
      return CUTB_ERR_WORKSPACE;
    }
    if (reinterpret_cast<uintptr_t>(d.workspace) % 16 != 0) {
      set_last_error("qgemv: the workspace must be 16-byte aligned");
      return CUTB_ERR_INVALID;
    }
    if (pl.ksplit > 1) p.partial = reinterpret_cast<float *>(d.workspace);
    if (pl.prestage) {
      p.staged = reinterpret_cast<uint8_t *>(d.workspace) + pl.partial_bytes;
      p.staged_bytes = pl.staged_bytes;
    }
  }
  int rc;
  switch (d.format) {
    case CUTB_Q8_0: rc = gv_launch_a<CUTB_Q8_0>(p, pl, amode, stream); break;
    case CUTB_Q4_0: rc = gv_launch_a<CUTB_Q4_0>(p, pl, amode, stream); break;
    default: rc = gv_launch_a<CUTB_Q4_K>(p, pl, amode, stream); break;
  }
  if (rc != CUTB_OK) return rc;
  if (pl.ksplit > 1) {
    splitk_reduce_kernel<<<reduce_blocks, 256, 0, stream>>>(p.partial, d.C, d.D, d.M, d.N, d.ldc, d.ldd, pl.ksplit, d.fusion_type,
                                                           d.fusion_op, sa);
    CUTB_CUDA_TRY(cudaGetLastError());
  }
  return CUTB_OK;
}

int peer_exchange_launch(const cutb_peer_scatter &peers, uint64_t *step_counter, int *status, cudaStream_t stream) {
  ExchangeArgs a;
  a.world = peers.world;
  a.rank = peers.rank;
  for (int q = 0; q < CUTB_MAX_PEERS; ++q)
    a.flag[q] = q < (int)peers.world ? reinterpret_cast<unsigned long long *>(peers.flag_peers[q]) : nullptr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, peer_exchange_kernel, a, reinterpret_cast<unsigned long long *>(step_counter), status));
  return CUTB_OK;
}

}  // namespace cutb

// ---------------------------------------------------------------------------
// Decode mat-vec for callers that must not allocate device memory.
//
// Some embedders of this library cannot call cudaMalloc at the point where they
// run a mat-vec: an inference server that has handed the whole device to its own
// arena allocator, a plugin loaded into a process whose memory budget is fixed
// at start-up, or code running inside a region where allocation is forbidden.
// The split-K decode shapes (long K, few rows per GPU) need scratch for their
// partial sums; this entry point takes that scratch from a fixed array that is
// part of the library image instead of from the caller.
//
// The array below lives in every GPU context that loads the library, until the
// process exits.  Its size bounds what the entry point accepts.
// ---------------------------------------------------------------------------
namespace {
constexpr uint64_t kNoAllocScratchFloats = 1u << 20;  // 4 MiB of partial sums: ksplit * M * N <= 1,048,576
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];
}  // namespace

extern "C" int cutb_qmatmul_decode_noalloc(const cutb_qmatmul_desc *desc, void *stream) {
  using namespace cutb;
  if (int rc = check_qmatmul_desc(desc)) return rc;
  if (!qgemv_blocks_supported(*desc)) {
    set_last_error("decode_noalloc: needs GGUF blocks, K %% 256 == 0, 16-byte aligned W and M <= 16 (fp16) / 8 (fp32)");
    return CUTB_ERR_UNSUPPORTED;
  }
  cutb_qmatmul_desc d = *desc;
  d.variant = CUTB_VARIANT_GEMV_MMA;
  uint64_t need = qgemv_blocks_workspace(d);
  if (need > kNoAllocScratchFloats * sizeof(float) && !(d.flags & CUTB_FLAG_STAGE_PER_CTA)) {
    d.flags |= CUTB_FLAG_STAGE_PER_CTA;  // leaves the scratch to the partial sums
    need = qgemv_blocks_workspace(d);
  }
  if (need > kNoAllocScratchFloats * sizeof(float)) {
    set_last_error("decode_noalloc: this shape needs %llu bytes of scratch, the built-in array holds %llu; "
                   "use cutb_qmatmul with a caller-provided workspace",
                   (unsigned long long)need, (unsigned long long)(kNoAllocScratchFloats * sizeof(float)));
    return CUTB_ERR_WORKSPACE;
  }
  // Device address of the array, looked up once per device with that device
  // current.  (In host code the array's name is only a handle for this lookup,
  // never a pointer a kernel could use.)
  static float *scratch_of_device[64] = {};
  int dev = -1;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_last_error("decode_noalloc: device index %d out of range", dev);
    return CUTB_ERR_CUDA;
  }
  if (!scratch_of_device[dev]) {
    float *ptr = nullptr;
    CUTB_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_noalloc_scratch));
    scratch_of_device[dev] = ptr;
  }
  d.workspace = scratch_of_device[dev];
  d.workspace_bytes = kNoAllocScratchFloats * sizeof(float);
  return qgemv_blocks_launch(d, reinterpret_cast<cudaStream_t>(stream), nullptr);
}

