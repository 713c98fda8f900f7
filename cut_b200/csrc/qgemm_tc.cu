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
// of activation stages (three at 512 tokens) and a ring of two weight tiles (three up to 256 tokens per CTA).
//
// Every wait is bounded; on expiry the CTA records CUTB_ERR_TIMEOUT in the
// caller's status word, skips its remaining work, frees its tensor memory and
// returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include "qgemm_tc_common.cuh"

namespace cutb {
namespace {

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
  // K stages: all of them, or this CTA's share when K is split over blockIdx.z (long K on few weight rows)
  const uint32_t nk_all = p.K / (TC_BK * KS), nk_per = (nk_all + p.ksplit - 1) / p.ksplit;
  const uint32_t kb = blockIdx.z * nk_per;                                     // first stage
  const uint32_t nk = kb < nk_all ? (kb + nk_per < nk_all ? nk_per : nk_all - kb) : 0;
  const uint32_t kc0 = kb * KS;                                                // first 64-k chunk
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
            tma_load_2d(dst + (sub * MB + mb) * TC_TILE_BYTES, &tmapA, (kc0 + ks * KS + sub) * TC_BK, m0 + mb * TC_BT, bar);
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
      if constexpr (tc_is_plane(FMT)) load_window_plane<FMT>(p, n, (kc0 + g * KS) * TC_BK, nxt);
      else load_window<FMT>(wrow, (kc0 + g * KS) * TC_BK, nxt);
    }
    // this group's slot sequence: start at slot g, advance by G modulo NB
    uint32_t sb = g % NB;
    uint32_t sc = 0, pc = 0;  // consumed barrier of stage ks - NB, once ks >= NB
    bool sc_set = false;
    for (uint32_t ks = g; ks < nk && !dead; ks += G) {
      uint8_t *slot = b_ring + sb * b_slot_bytes;
      for (uint32_t sub = 0; sub < KS; ++sub) {
        const uint32_t chunk = kc0 + ks * KS + sub;  // 64-k chunk of the row
        const RawWindow<FMT> cur = nxt;
        // the chunk this thread converts next: the following sub-tile, or the first of the group's next stage
        const uint32_t nchunk = sub + 1 < KS ? chunk + 1 : kc0 + (ks + G) * KS;
        if (live && nchunk < kc0 + nk * KS) {
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
          if (p.ksplit > 1) {  // this CTA's share of K: raw sums to its plane of the workspace; tc_splitk_reduce_kernel finishes
            float *dstp = p.partial + ((size_t)blockIdx.z * p.M + mbase) * p.N + nn;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n_ok && mbase + i < p.M) dstp[(size_t)i * p.N] = __uint_as_float(v[i]);
            continue;
          }
          if (p.glu) {
            // gate and up rows are neighbouring lanes: the even lane takes its partner's accumulator, applies the
            // gate's activation to its own and stores one output column for the pair
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              float x[8], up[8], dd[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                x[i] = __uint_as_float(v[8 * g8 + i]);
                up[i] = __shfl_xor_sync(0xffffffffu, x[i], 1);
                dd[i] = 0.f;
              }
              apply_epilogue_n<8>(x, dd, CUTB_FUSION_UNARY, p.fusion_op);
              if (n_ok && !(lane & 1u)) {
                float *dstp = p.C + (size_t)mbase * p.ldc + (nn >> 1);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (mbase + 8 * g8 + i < p.M) dstp[(size_t)(8 * g8 + i) * p.ldc] = x[i] * up[i];
              }
            }
            continue;
          }
          float *dst = p.C + (size_t)mbase * p.ldc + nn;
          if (p.fusion_type == CUTB_FUSION_NONE) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n_ok && mbase + i < p.M) dst[(size_t)i * p.ldc] = __uint_as_float(v[i]);
          } else {
            // eight values at a time, the op selected once per group (apply_epilogue_n) rather than once per value;
            // small groups keep the fused path from setting the kernel's register allocation
            const float *dsrc = p.fusion_type == CUTB_FUSION_BINARY ? p.D + (size_t)mbase * p.ldd + nn : nullptr;
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              float x[8], dd[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                x[i] = __uint_as_float(v[8 * g8 + i]);
                dd[i] = (dsrc && n_ok && mbase + 8 * g8 + i < p.M) ? dsrc[(size_t)(8 * g8 + i) * p.ldd] : 0.f;
              }
              apply_epilogue_n<8>(x, dd, p.fusion_type, p.fusion_op);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (n_ok && mbase + 8 * g8 + i < p.M) dst[(size_t)(8 * g8 + i) * p.ldc] = x[i];
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

// K split: the planes of partial sums added in a fixed order, then the fused epilogue (paired rows included).
__global__ void tc_splitk_reduce_kernel(const TcParams p) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)p.M * p.N;
  float sum = 0.f;
  uint32_t m = 0, n = 0;
  const bool in = idx < total;
  if (in) {
    m = (uint32_t)(idx / p.N), n = (uint32_t)(idx % p.N);
    for (uint32_t z = 0; z < p.ksplit; ++z) sum += p.partial[(size_t)z * total + idx];
  }
  if (p.glu) {  // gate and up columns sit in neighbouring threads (N is even, so a pair never straddles a row)
    const float up = __shfl_xor_sync(0xffffffffu, sum, 1);
    if (in && !(n & 1u)) p.C[(size_t)m * p.ldc + (n >> 1)] = apply_epilogue(sum, CUTB_FUSION_UNARY, p.fusion_op, 0.f) * up;
    return;
  }
  if (!in) return;
  const float dv = p.fusion_type == CUTB_FUSION_BINARY ? p.D[(size_t)m * p.ldd + n] : 0.f;
  p.C[(size_t)m * p.ldc + n] = apply_epilogue(sum, p.fusion_type, p.fusion_op, dv);
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
  dim3 grid((p.N + TC_BW - 1) / TC_BW, (p.M + p.mb * TC_BT - 1) / (p.mb * TC_BT), p.ksplit);
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

namespace {
// Token blocks per CTA and K split.  Few weight rows (a 4096-row projection is 32 column tiles) would leave most SMs
// idle at 512 tokens per CTA.  With a long K (the down projection, K = 14336) the K stages are shared out over
// blockIdx.z instead: every weight is still dequantised once, 512 tokens amortise it, and the partial sums meet in
// the workspace (512 x 14336 x 4096: 112 us with 128 tokens per CTA).  Otherwise fewer tokens per CTA until the grid
// covers at least half of the SMs: each weight tile is then dequantised once per token group, which costs far less
// than the idle SMs.
void tc_shape_plan(const cutb_qmatmul_desc &d, uint32_t sm_count, uint32_t *mb_out, uint32_t *ksplit_out) {
  const uint32_t mblocks = (d.M + TC_BT - 1) / TC_BT, ctiles = (d.N + TC_BW - 1) / TC_BW;
  uint32_t mb = mblocks < TC_MAX_MB ? mblocks : TC_MAX_MB, ksplit = 1;
  const uint32_t ctas = ctiles * ((mblocks + mb - 1) / mb);
  const uint32_t nk_all = d.K / TC_BK;  // (such CTAs run 64-k stages)
  // (K = 4096 measured no better split than not: 512 x 4096 x 4096 35.3 against 36.2 us, 6144 rows 51 against 38)
  if (mb == TC_MAX_MB && d.K >= 8192 && ctas * 2 <= sm_count) {
    uint32_t want = sm_count / ctas;
    if (want > 8) want = 8;
    const uint32_t per = (nk_all + want - 1) / want;
    ksplit = (nk_all + per - 1) / per;  // no empty share
  } else {
    while (mb > 1 && ctiles * ((mblocks + mb - 1) / mb) * 2 <= sm_count) mb = (mb + 1) / 2;
  }
  *mb_out = mb;
  *ksplit_out = ksplit;
}
uint64_t tc_cast_bytes(const cutb_qmatmul_desc &d) {
  return d.a_dtype == CUTB_F32 ? (((uint64_t)d.M * d.K * sizeof(__half) + 15) & ~(uint64_t)15) : 0;
}
}  // namespace

uint64_t qgemm_tc_workspace(const cutb_qmatmul_desc &d) {
  if (qgemm_skinny_applies(d)) return qgemm_skinny_workspace(d);
  // fp32 activations are rounded to fp16 rows of K elements first; a K split adds its planes of partial sums
  DeviceInfo di;
  const uint32_t sms = get_device_info(&di) == CUTB_OK ? (uint32_t)di.sm_count : 148u;
  uint32_t mb, ksplit;
  tc_shape_plan(d, sms, &mb, &ksplit);
  return tc_cast_bytes(d) + (ksplit > 1 ? (uint64_t)ksplit * d.M * d.N * sizeof(float) : 0);
}

int qgemm_tc_launch(const cutb_qmatmul_desc &d, cudaStream_t stream) {
  if (qgemm_skinny_applies(d)) return qgemm_skinny_launch(d, stream);
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
  p.glu = (d.flags & CUTB_FLAG_GLU_PAIRS) ? 1 : 0;
  p.status = d.status;
  p.S = reinterpret_cast<const uint16_t *>(d.scales);
  p.ldb = d.ldb;
  p.lds = d.lds;
  p.blocksK = (d.K + 31) / 32;
  tc_shape_plan(d, (uint32_t)di.sm_count, &p.mb, &p.ksplit);
  const uint64_t cast_bytes = tc_cast_bytes(d), partial_bytes = p.ksplit > 1 ? (uint64_t)p.ksplit * d.M * d.N * sizeof(float) : 0;
  p.partial = nullptr;
  if (p.ksplit > 1) {
    // without room for the partial sums: the tokens-per-CTA rule (a K split of one never asks for any)
    if (!d.workspace || d.workspace_bytes < cast_bytes + partial_bytes || reinterpret_cast<uintptr_t>(d.workspace) % 16 != 0) {
      const uint32_t mblocks = (d.M + TC_BT - 1) / TC_BT, ctiles = (d.N + TC_BW - 1) / TC_BW;
      p.ksplit = 1;
      while (p.mb > 1 && ctiles * ((mblocks + p.mb - 1) / p.mb) * 2 <= (uint32_t)di.sm_count) p.mb = (p.mb + 1) / 2;
    } else {
      p.partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d.workspace) + cast_bytes);
    }
  }
  // weight slots: two (one per converter group) when the activation stages need the room; up to 256 tokens per
  // CTA a third one loosens the hand-off chain converter -> issuer -> tensor core -> converter (512 x 4096 x 4096
  // 39.1 -> 36.5 us, 512 x 14336 x 4096 121.4 -> 112.4 us; no change with four); the rest of shared memory holds
  // activation stages in flight
  p.nb = p.mb <= 2 ? 3 : 2;
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
    const uint64_t need = cast_bytes;
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
  int rc;
  if (d.layout == CUTB_LAYOUT_KN_PLANES) {
    if (d.format == CUTB_Q8_0) rc = tc_launch<TC_PLANE_Q8>(map, p, stream);
    else rc = d.affine ? tc_launch<TC_PLANE_Q4A>(map, p, stream) : tc_launch<TC_PLANE_Q4>(map, p, stream);
  } else {
    switch (d.format) {
      case CUTB_Q8_0: rc = tc_launch<CUTB_Q8_0>(map, p, stream); break;
      case CUTB_Q4_0: rc = tc_launch<CUTB_Q4_0>(map, p, stream); break;
      default: rc = tc_launch<CUTB_Q4_K>(map, p, stream); break;
    }
  }
  if (rc != CUTB_OK || p.ksplit <= 1) return rc;
  const size_t total = (size_t)d.M * d.N;
  tc_splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(p);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace cutb
