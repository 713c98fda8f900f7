// Tensor-core GEMM over native GGUF blocks for 1 < M <= 128 tokens (batched decode, short prefill).
//
// C[M, N] = epilogue(A[M, K] * dequant(W)^T).  Same contract and arithmetic as the prefill GEMM (fp16
// operands, the dequantised weight rounded to fp16 as the reference's tensor-core variants round it,
// MatMulQ4CoopMatTiled.cu:84-87 / MatMulQ8CoopMatTiled.cu:71-74; fp32 accumulation), but the operand roles
// are the other way round.  In the prefill kernel (weights = the MMA's M operand, tokens = its N operand) the
// issuer spent the same 95-140 cycles per tcgen05.mma with 32 tokens as with 256, so with few tokens almost all
// of an instruction is empty.  Here the tokens are the M operand (one token per tensor-memory lane, 128 lanes,
// only the rows that exist are loaded) and 256 weight rows are the N operand: one instruction covers twice the
// weights, and the accumulator comes back token-major, so a thread of the epilogue stores 32 consecutive output
// columns of its token.
//
// Few tokens mean few tiles, so every SM must be given work: the 256-k units of all weight tiles are numbered
// tile by tile and dealt in equal contiguous runs to one CTA per SM (stream-K).  A CTA touches at most two
// tiles; each accumulates in its own 256 tensor-memory columns.  A tile whose K a CTA covered whole is finished
// there (fused epilogue, written to C); a shared tile goes raw to the CTA's head / tail slot in the workspace
// and tc_skinny_fixup_kernel adds the slots in CTA order and applies the epilogue (fixed summation order for a
// shape and a device).
//
//   warp 0      allocates tensor memory; one lane issues the MMAs of every 64-k stage and commits them to the
//               stage's "consumed" barrier (frees the activation stage and the fp16 weight slot)
//   warp 1      one lane issues the TMA tensor copies of the activation rows (64 k x tokens, fp16,
//               128-byte swizzle, no cluster multicast)
//   warp 2      block formats: one lane issues the TMA copies of raw weight granules (64 rows x 256 k of block
//               bytes, a 2-D tensor map over the weight, no swizzle, no multicast) into a ring
//   warps 4-19  block formats: two converter groups of 256 threads, one weight row per thread; a group widens
//               every other 64-k stage from the raw granule (conflict-free 16-byte shared loads, half2
//               arithmetic) into the K-major, 128-byte-swizzled fp16 slot.  Plane formats: warps 4-11, one
//               group, raw bytes of the next chunk in flight in registers as in the prefill kernel.
//               The same warps run the epilogue (tcgen05.ld, lane = token, 32 columns = 32 weight rows).
// Programmatic dependent launch: the kernel lets its successor start at once and waits for its predecessor only
// before the first activation copy and before the first store.  Every wait is bounded; on expiry the CTA records
// CUTB_ERR_TIMEOUT, drains its copies, frees its tensor memory and returns.
#include "qgemm_tc_common.cuh"

namespace cutb {
namespace {

constexpr int SK_BW = 256;                                // weight rows per tile (MMA N)
constexpr int SK_CONV_THREADS = SK_BW;                    // one row per converter thread of a group
// Converter groups: group c of C converts the 64-k stages c, c + C, ... of every unit, so that the dependent
// load -> widen -> store chains of C stages overlap (16 warps hide what 8 cannot).  The plane formats keep one
// group: their converters hold the next chunk's bytes in registers and need the whole register file.
__host__ __device__ constexpr int sk_conv_groups(int fmt) { return tc_is_plane(fmt) ? 1 : 2; }
__host__ __device__ constexpr int sk_threads(int fmt) { return TC_CTRL_THREADS + SK_CONV_THREADS * sk_conv_groups(fmt); }
constexpr uint32_t SK_W_TILE_BYTES = SK_BW * TC_BK * 2;   // 32 KB: 256 rows x 64 k of fp16
constexpr uint32_t SK_UNIT_K = 256;                       // k per unit of work: one raw granule row, four 64-k stages
constexpr uint32_t SK_SUBS = SK_UNIT_K / TC_BK;
constexpr uint32_t SK_GRAN_ROWS = 64;                     // weight rows per raw granule
constexpr uint32_t SK_GRANS = SK_BW / SK_GRAN_ROWS;       // granules per unit

// bytes of 256 k of one weight row in the GGUF block formats (a multiple of 16 in all three)
__host__ __device__ constexpr uint32_t sk_row_chunk_bytes(int fmt) {
  return fmt == CUTB_Q8_0 ? 8u * 34u : 144u;  // Q4_0: 8 blocks of 18; Q4_K: one super-block
}

struct SkParams {
  const uint8_t *W;
  uint64_t row_bytes;
  float *C;
  uint32_t ldc;
  const float *D;
  uint32_t ldd;
  uint32_t M, K, N;
  uint32_t bt;        // token rows loaded per stage (M rounded up to 8; the MMA always spans 128 lanes)
  uint32_t sa, nb;    // activation stages and fp16 weight slots in shared memory (64 k each)
  uint32_t rs;        // raw granules in shared memory (block formats)
  uint32_t tiles;     // weight tiles of 256 rows
  uint32_t per;       // units (256 k of one tile) per CTA
  uint32_t tmem_cols;
  int fusion_type, fusion_op;
  int glu;  // rows in (gate, up) pairs: C[m, n / 2] = unary(acc[m, n]) * acc[m, n + 1], n even
  int *status;
  float *partial;     // stream-K slots [2 * CTAs][bt][256]
  int vec_ok;         // C (and D) rows allow 16-byte accesses
  // the reference's [K, N] plane layout (TC_PLANE_* formats)
  const uint16_t *S;
  uint32_t ldb, lds, blocksK;
};

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// The aligned 16-byte lines around 64-k chunk `sub` of a raw granule row in shared memory (same window as the
// global-memory loader: a granule row starts on a 256-k boundary of the weight row, 16-byte aligned).
template <int FMT> __device__ __forceinline__ void load_window_smem(uint32_t row, uint32_t sub, RawWindow<FMT> &r) {
  if constexpr (FMT == CUTB_Q4_K) {
    r.v[0] = lds_v4(row);
    r.v[1] = lds_v4(row + 16 + 32 * sub);
    r.v[2] = lds_v4(row + 32 + 32 * sub);
  } else {
    const uint32_t q = row + ((sub * 2 * block_bytes(FMT)) & ~15u);
#pragma unroll
    for (int i = 0; i < RawWindow<FMT>::NV; ++i) r.v[i] = lds_v4(q + 16 * i);
  }
}

template <int FMT>
__global__ void __launch_bounds__(sk_threads(FMT), 1)
    qgemm_skinny_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapW, const SkParams p) {
  constexpr bool RAW = !tc_is_plane(FMT);  // block formats: raw bytes staged by the copy engine
  constexpr uint32_t CHUNK = RAW ? sk_row_chunk_bytes(FMT) : 0u, GRAN_BYTES = SK_GRAN_ROWS * CHUNK;
  constexpr uint32_t CG = sk_conv_groups(FMT);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t SA = p.sa, NB = p.nb, RS = p.rs, BT = p.bt;
  // Activation tiles are packed at the rows that exist; the MMA reads 128 rows from a tile's base, so the rows
  // past BT are whatever follows in shared memory (the next tile, or the weight ring behind the activation ring):
  // they only reach accumulator lanes that nobody reads.
  const uint32_t a_tile_bytes = BT * 128u;
  uint8_t *a_ring = smem;
  uint8_t *b_ring = smem + ((SA * a_tile_bytes + 1023u) & ~1023u);
  uint8_t *raw_ring = b_ring + NB * SK_W_TILE_BYTES;
  const uint32_t NC = SA + NB;  // ring of "consumed" barriers, one per 64-k stage in flight
  // fullA[SA] fullB[NB] consumed[NC] accum rawfull[RS] rawempty[RS]
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw_ring + RS * GRAN_BYTES);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * SA + 2 * NB + 1 + 2 * RS);
  uint32_t *abort_flag = tmem_slot + 1;

  // Programmatic dependent launch: this kernel waits for the kernel before it only where it first touches what that
  // kernel may have written (activations, C, D).  Without the K split the next kernel of the stream may start its
  // prologue at once.  With it the next kernel is the fix-up, whose blocks would become resident wherever an SM has
  // room and sit there until this grid is done -- which keeps the CTAs of the GEMM after it off those SMs (a trace
  // showed a fifth of them entering 8 us late and the grid ending 5 us after its median CTA); so the trigger moves
  // to the end of the CTA.
  if (!p.partial) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t nk = p.K / SK_UNIT_K;  // units of one tile
  // this CTA's run of units: [u0, u0 + nunits), numbered tile by tile
  const uint32_t total = p.tiles * nk, u0 = blockIdx.x * p.per;
  const uint32_t nunits = u0 < total ? (u0 + p.per < total ? p.per : total - u0) : 0;
  const uint32_t tile0 = u0 / nk, k_first = u0 % nk;
  const uint32_t nsegs = nunits ? (k_first + nunits - 1) / nk + 1 : 0;  // tiles touched (at most 2)
  const uint32_t nstages = nunits * SK_SUBS;
  const uint32_t fulla_u = smem_u32(bars), fullb_u = fulla_u + SA * 8, cons_u = fullb_u + NB * 8, accum_u = cons_u + NC * 8;
  const uint32_t rawfull_u = accum_u + 8, rawempty_u = rawfull_u + RS * 8;

  if (tid == 0) {
    for (uint32_t s = 0; s < SA; ++s) mbar_init(fulla_u + s * 8, 1);                     // the TMA lane's arrive.expect_tx
    for (uint32_t s = 0; s < NB; ++s) mbar_init(fullb_u + s * 8, SK_CONV_THREADS / 32);  // one arrival per converter warp
    for (uint32_t s = 0; s < NC; ++s) mbar_init(cons_u + s * 8, 1);                      // the issuer's tcgen05.commit
    mbar_init(accum_u, 1);
    for (uint32_t s = 0; s < RS; ++s) {
      mbar_init(rawfull_u + s * 8, 1);                    // the raw producer's arrive.expect_tx
      mbar_init(rawempty_u + s * 8, CG * SK_GRAN_ROWS / 32);  // the converter warps that read the granule
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(p.tmem_cols)
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
    // ---- MMA issuer ----------------------------------------------------------------------
    if (lane == 0 && nunits) {
      const uint64_t proto = umma_desc_sw128(0);
      const uint32_t desc_hi = (uint32_t)(proto >> 32), lo0 = (uint32_t)proto;
      const uint32_t w_lo0 = lo0 + ((smem_u32(b_ring) & 0x3FFFFu) >> 4), t_lo0 = lo0 + ((smem_u32(a_ring) & 0x3FFFFu) >> 4);
      const uint32_t idesc = umma_idesc_f16(128, SK_BW);  // M = 128 token lanes, N = 256 weight rows
      const uint32_t a_tile_desc = a_tile_bytes >> 4, w_tile_desc = SK_W_TILE_BYTES >> 4;
      uint32_t sa = 0, pa = 0, sb = 0, pb = 0, sc = 0;
      uint32_t left = (nk - k_first) * SK_SUBS;  // stages until the next tile begins
      uint32_t d = tmem_base, acc = 0;           // acc 0: the next MMA starts a tile's accumulator
      bool dead = false;
      for (uint32_t j = 0; j < nstages; ++j) {
        if (!mbar_spin_bounded(fullb_u + sb * 8, pb) || !mbar_spin_bounded(fulla_u + sa * 8, pa)) {
          give_up();
          dead = true;
          break;
        }
        tc_fence_after();
        const uint32_t t_lo = t_lo0 + sa * a_tile_desc, w_lo = w_lo0 + sb * w_tile_desc;
        // 16 k = 32 bytes = 2 descriptor units along the swizzled row
        umma_f16(d, t_lo, w_lo, desc_hi, idesc, acc);
        umma_f16(d, t_lo + 2, w_lo + 2, desc_hi, idesc, 1);
        umma_f16(d, t_lo + 4, w_lo + 4, desc_hi, idesc, 1);
        umma_f16(d, t_lo + 6, w_lo + 6, desc_hi, idesc, 1);
        acc = 1;
        umma_commit(cons_u + sc * 8);  // the stage is consumed when these MMAs have read it
        if (++sa == SA) sa = 0, pa ^= 1u;
        if (++sb == NB) sb = 0, pb ^= 1u;
        if (++sc == NC) sc = 0;
        if (--left == 0) left = nk * SK_SUBS, d += SK_BW, acc = 0;  // the next tile's columns
      }
      if (!dead) umma_commit(accum_u);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- TMA producer: the activation rows of every 64-k stage ------------------------------
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations may come from the kernel before
      uint32_t sa = 0, pa = 1u;  // parity of the slot's previous fill (used when draining)
      uint32_t sc = 0, pc = 0;   // consumed barrier of stage j - SA
      uint32_t issued = 0, kc = k_first * SK_SUBS;  // 64-k chunk of the row
      const uint32_t a_base = smem_u32(a_ring);
      for (uint32_t j = 0; j < nstages; ++j) {
        if (j >= SA) {
          // rings ahead of the issuer: a parked wait costs nothing here and leaves the issue slots to the converters
          if (!mbar_wait_probe_first(cons_u + sc * 8, pc)) {
            give_up();
            break;
          }
          if (++sc == NC) sc = 0, pc ^= 1u;
        }
        if (aborted()) break;
        const uint32_t bar = fulla_u + sa * 8;
        mbar_arrive_expect_tx(bar, a_tile_bytes);
        tma_load_2d(a_base + sa * a_tile_bytes, &tmapA, kc * TC_BK, 0, bar);
        ++issued;
        if (++sa == SA) sa = 0, pa ^= 1u;
        if (++kc == nk * SK_SUBS) kc = 0;
      }
      if (aborted()) {  // no copy may still be landing when the CTA retires
        const uint32_t pending = issued < SA ? issued : SA;
        for (uint32_t i = 0; i < pending; ++i) {
          if (sa == 0) sa = SA, pa ^= 1u;
          --sa;
          mbar_wait_bounded(fulla_u + sa * 8, pa ^ 1u, 1u << 10);
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ---- raw producer: the unit's granules (64 weight rows x 256 k of raw block bytes each) follow one another through
    // a ring as deep as shared memory allows: the bytes in flight per SM are what sets the streaming rate.  Rows past
    // N are zero-filled by the copy engine and dequantise to zero.  Weights are constants: no wait for the kernel before ----
    if constexpr (RAW) {
      if (lane == 0) {
        uint32_t slot = 0, ph = 1, issued = 0;  // ph: parity of the slot's previous "empty" phase
        uint32_t a = k_first, tile = tile0;
        const uint32_t raw_base = smem_u32(raw_ring);
        for (uint32_t g = 0; g < SK_GRANS * nunits; ++g) {
          if (g >= RS) {
            if (!mbar_wait_probe_first(rawempty_u + slot * 8, ph)) {
              give_up();
              break;
            }
          }
          if (aborted()) break;
          const uint32_t bar = rawfull_u + slot * 8;
          mbar_arrive_expect_tx(bar, GRAN_BYTES);
          tma_load_2d(raw_base + slot * GRAN_BYTES, &tmapW, a * (CHUNK / 4), tile * SK_BW + (g % SK_GRANS) * SK_GRAN_ROWS, bar);
          ++issued;
          if (++slot == RS) slot = 0, ph ^= 1u;  // first turn waits for nothing; second turn for phase 0, ...
          if (g % SK_GRANS == SK_GRANS - 1) {
            if (++a == nk) a = 0, ++tile;
          }
        }
        if (aborted()) {
          // drain: every granule issued completes its "full" phase; wait (bounded) for the last ring turn
          const uint32_t pending = issued < RS ? issued : RS;
          for (uint32_t i = 0; i < pending; ++i) {
            const uint32_t g = issued - 1 - i;
            mbar_wait_bounded(rawfull_u + (g % RS) * 8, (g / RS) & 1u, 1u << 10);
          }
        }
      }
      __syncwarp();
    }
  } else if (warp >= 4) {
    // ---- converters: one of the tile's 256 weight rows per thread ---------------------------
    const uint32_t ct = tid - TC_CTRL_THREADS, r = ct % SK_CONV_THREADS, grp = ct / SK_CONV_THREADS;
    const uint32_t h = r / SK_GRAN_ROWS, rr = r % SK_GRAN_ROWS;
    bool dead = false;
    RawWindow<FMT> nxt;
#pragma unroll
    for (int i = 0; i < RawWindow<FMT>::NV; ++i) nxt.v[i] = make_uint4(0, 0, 0, 0);
    // plane layout: raw bytes of 64-k chunk `sub` of this CTA's unit i straight from global memory, one chunk ahead
    auto fetch = [&](uint32_t i, uint32_t sub, RawWindow<FMT> &w) {
      if constexpr (!RAW) {
        const uint32_t a = k_first + i, n = (tile0 + a / nk) * SK_BW + r, k0 = ((a % nk) * SK_SUBS + sub) * TC_BK;
        if (n < p.N) load_window_plane<FMT>(p, n, k0, w);
      }
    };
    if (nunits) fetch(0, 0, nxt);
    // shared-window offsets of this row's eight 16-byte chunks in a swizzled fp16 tile
    uint32_t soff[8];
#pragma unroll
    for (uint32_t c = 0; c < 8; ++c) soff[c] = r * 128u + ((c ^ (r & 7u)) << 4);
    const uint32_t b_base = smem_u32(b_ring), raw_row0 = smem_u32(raw_ring) + rr * CHUNK;
    // Ring positions advance without divisions: this group's stages are j = grp, grp + CG, ...; its fp16 slot is
    // j mod NB, the barrier it waits on is that of stage j - NB (index mod NC, phase flipping per turn); its
    // granules are g = h, h + SK_GRANS, ... (slot g mod RS, phase flipping per turn; RS >= SK_GRANS).
    uint32_t j = grp, sb = grp % NB;
    uint32_t cidx = 0, cph = 0;
    {
      uint32_t j0 = grp;  // first stage that has a predecessor in its slot
      while (j0 < NB) j0 += CG;
      cidx = j0 - NB;
    }
    uint32_t rslot = h % RS, rph = 0;
    uint32_t kl = k_first, tile = tile0;
    for (uint32_t i = 0; i < nunits && !dead; ++i) {
      const bool live = RAW || tile * SK_BW + r < p.N;
      const uint32_t rawrow = raw_row0 + rslot * GRAN_BYTES;
      if constexpr (RAW) {
        uint32_t ok = 1;
        if (lane == 0) ok = mbar_spin_bounded(rawfull_u + rslot * 8, rph) ? 1u : 0u;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) give_up();
          dead = true;
          break;
        }
      }
#pragma unroll 1
      for (uint32_t sub = grp; sub < SK_SUBS; sub += CG, j += CG) {
        RawWindow<FMT> cur;
        if constexpr (RAW) {
          load_window_smem<FMT>(rawrow, sub, cur);
        } else {
          cur = nxt;
          if (sub + 1 < SK_SUBS) fetch(i, sub + 1, nxt);
          else if (i + 1 < nunits) fetch(i + 1, 0, nxt);
        }
        uint4 out[8];
        if (live) {
          if constexpr (RAW) convert_window<FMT>(cur, (kl * SK_SUBS + sub) * TC_BK, out);
          else convert_window_plane<FMT>(cur, out);
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
        uint32_t ok = 1;  // one lane per warp polls the barrier
        if (j >= NB) {  // the slot's previous stage j - NB must have been consumed
          if (lane == 0) ok = mbar_spin_bounded(cons_u + cidx * 8, cph) ? 1u : 0u;
          cidx += CG;
          if (cidx >= NC) cidx -= NC, cph ^= 1u;
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
        const uint32_t tile_u = b_base + sb * SK_W_TILE_BYTES;
#pragma unroll
        for (int c = 0; c < 8; ++c) sts_v4(tile_u + soff[c], out[c]);
        fence_async_smem();  // make the generic-proxy stores visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(fullb_u + sb * 8);
        sb += CG;
        if (sb >= NB) sb -= NB;
      }
      if (dead) break;
      if constexpr (RAW) {
        __syncwarp();  // every lane has read its row of the granule
        if (lane == 0) mbar_arrive(rawempty_u + rslot * 8);
        rslot += SK_GRANS;
        if (rslot >= RS) rslot -= RS, rph ^= 1u;
      }
      if (++kl == nk) kl = 0, ++tile;
    }

    // ---- epilogue: lane = token; warp w reads the lane quarter w % 4 and shares its 32-column
    // items with the other warp of that quarter ----
    const uint32_t q = warp & 3, half = (warp - 4) >> 2;  // warps of one quarter share its items
    const uint32_t m = q * 32 + lane;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // C, D and the workspace may still be in use by the kernel before
    if (!dead && !aborted() && nunits && q * 32 < p.M) {
      if (!mbar_wait_bounded(accum_u, 0)) {
        give_up();
      } else {
        tc_fence_after();
        constexpr uint32_t per_seg = SK_BW / 32;
#pragma unroll 1
        for (uint32_t item = half; item < nsegs * per_seg; item += 2 * CG) {
          const uint32_t seg = item / per_seg, c0 = (item % per_seg) * 32;
          const uint32_t k_lo = seg == 0 ? k_first : 0u;
          const uint32_t k_hi = seg + 1 == nsegs ? (k_first + nunits - 1) % nk + 1 : nk;
          const bool whole = k_lo == 0 && k_hi == nk;
          uint32_t v[32];
          tmem_ld32(tmem_base + ((q * 32) << 16) + seg * SK_BW + c0, v);
          if (m >= p.M) continue;
          if (!whole) {
            float4 *dst = reinterpret_cast<float4 *>(p.partial + ((size_t)(2 * blockIdx.x + (seg ? 1u : 0u)) * BT + m) * SK_BW + c0);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]),
                                   __uint_as_float(v[4 * i + 3]));
            continue;
          }
          const uint32_t n = (tile0 + seg) * SK_BW + c0;
          if (n >= p.N) continue;
          if (p.glu) {
            // gate and up rows are neighbouring columns of this token: 16 outputs from the thread's 32 accumulators
            float *dstp = p.C + (size_t)m * p.ldc + (n >> 1);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              float x[8], up[8], dd[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                x[i] = __uint_as_float(v[16 * hh + 2 * i]);
                up[i] = __uint_as_float(v[16 * hh + 2 * i + 1]);
                dd[i] = 0.f;
              }
              apply_epilogue_n<8>(x, dd, CUTB_FUSION_UNARY, p.fusion_op);
              if (p.vec_ok && n + 32 <= p.N) {
                reinterpret_cast<float4 *>(dstp)[2 * hh] = make_float4(x[0] * up[0], x[1] * up[1], x[2] * up[2], x[3] * up[3]);
                reinterpret_cast<float4 *>(dstp)[2 * hh + 1] = make_float4(x[4] * up[4], x[5] * up[5], x[6] * up[6], x[7] * up[7]);
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (n + 16 * hh + 2 * i < p.N) dstp[8 * hh + i] = x[i] * up[i];
              }
            }
            continue;
          }
          float *dst = p.C + (size_t)m * p.ldc + n;
          const float *dsrc = p.fusion_type == CUTB_FUSION_BINARY ? p.D + (size_t)m * p.ldd + n : nullptr;
          const bool vec = p.vec_ok && n + 32 <= p.N;
          // 16 values at a time, the fused op selected once per group (apply_epilogue_n), not once per value
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            float x[16], dd[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = __uint_as_float(v[16 * hh + i]);
            if (p.fusion_type != CUTB_FUSION_NONE) {
              if (dsrc && vec) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float4 t = __ldg(reinterpret_cast<const float4 *>(dsrc) + 4 * hh + i);
                  dd[4 * i] = t.x, dd[4 * i + 1] = t.y, dd[4 * i + 2] = t.z, dd[4 * i + 3] = t.w;
                }
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) dd[i] = (dsrc && n + 16 * hh + i < p.N) ? dsrc[16 * hh + i] : 0.f;
              }
              apply_epilogue_n<16>(x, dd, p.fusion_type, p.fusion_op);
            }
            if (vec) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<float4 *>(dst)[4 * hh + i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (n + 16 * hh + i < p.N) dst[16 * hh + i] = x[i];
            }
          }
        }
      }
    }
  }

  if (p.partial) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // release the tensor memory once every reader is done with it
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
  }
}

// A tile whose units were shared by several CTAs is the sum of their head / tail slots, added in CTA order,
// followed by the fused epilogue.  grid = (tiles, groups of SK_FIX_ROWS tokens), one thread per column.
constexpr uint32_t SK_FIX_ROWS = 4;
__global__ void __launch_bounds__(SK_BW) tc_skinny_fixup_kernel(const SkParams p, uint32_t nk) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the slots come from the GEMM kernel before
  const uint32_t t = blockIdx.x, c = threadIdx.x;
  const uint32_t c_first = t * nk / p.per, c_last = ((t + 1) * nk - 1) / p.per;
  if (c_first == c_last) return;  // one CTA covered the tile and wrote it
  const uint32_t n = t * SK_BW + c;
  const bool in_n = n < p.N;  // (the slots are 256 columns wide whatever N is; only the stores look at it)
  const uint32_t head_tile_first = (c_first * p.per) / nk;  // only the first sharer can have begun in an earlier tile
  const uint32_t m0 = blockIdx.y * SK_FIX_ROWS;
  float sum[SK_FIX_ROWS];
#pragma unroll
  for (uint32_t mm = 0; mm < SK_FIX_ROWS; ++mm) sum[mm] = 0.f;
  for (uint32_t cta = c_first; cta <= c_last; ++cta) {
    const uint32_t tail = (cta == c_first && head_tile_first != t) ? 1u : 0u;  // not the CTA's first tile
    const float *slot = p.partial + ((size_t)(2 * cta + tail) * p.bt + m0) * SK_BW + c;
#pragma unroll
    for (uint32_t mm = 0; mm < SK_FIX_ROWS; ++mm)  // the rows' loads are independent of one another
      if (m0 + mm < p.M) sum[mm] += slot[(size_t)mm * SK_BW];
  }
  if (p.glu) {  // gate and up columns sit in neighbouring threads; the even one stores the pair's output
#pragma unroll
    for (uint32_t mm = 0; mm < SK_FIX_ROWS; ++mm) {
      const float up = __shfl_xor_sync(0xffffffffu, sum[mm], 1);
      if (in_n && !(c & 1u) && m0 + mm < p.M)
        p.C[(size_t)(m0 + mm) * p.ldc + (n >> 1)] = apply_epilogue(sum[mm], CUTB_FUSION_UNARY, p.fusion_op, 0.f) * up;
    }
    return;
  }
#pragma unroll
  for (uint32_t mm = 0; mm < SK_FIX_ROWS; ++mm) {
    const uint32_t m = m0 + mm;
    if (m >= p.M || !in_n) break;
    const float dv = p.fusion_type == CUTB_FUSION_BINARY ? p.D[(size_t)m * p.ldd + n] : 0.f;
    p.C[(size_t)m * p.ldc + n] = apply_epilogue(sum[mm], p.fusion_type, p.fusion_op, dv);
  }
}

size_t sk_smem_bytes(int fmt, bool planes, uint32_t bt, uint32_t sa, uint32_t nb, uint32_t rs) {
  const size_t a_ring = ((size_t)sa * bt * 128 + 1023) & ~(size_t)1023;
  const size_t raw = planes ? 0 : (size_t)rs * SK_GRAN_ROWS * sk_row_chunk_bytes(fmt);
  return 1024 + a_ring + (size_t)nb * SK_W_TILE_BYTES + raw + (2 * sa + 2 * nb + 1 + 2 * rs) * 8 + 16;
}

struct SkPlan {
  uint32_t bt, sa, nb, rs, tiles, per, grid, tmem_cols;
  bool split;
  uint64_t cast_bytes, partial_bytes;
};

bool sk_plan(const cutb_qmatmul_desc &d, uint32_t sm_count, size_t smem_optin, bool allow_split, SkPlan *pl) {
  const bool planes = d.layout == CUTB_LAYOUT_KN_PLANES;
  pl->bt = ((d.M + 7) / 8) * 8;  // whole 8-row swizzle groups
  pl->tiles = (d.N + SK_BW - 1) / SK_BW;
  // Shared memory.  Three fp16 slots measured 12 % faster than two (the slot hand-off chain converter -> issuer ->
  // tensor core -> converter is what a stage waits on), about 32 KB of activation stages, and the raw ring takes
  // every granule that still fits (at least one unit's).  Planes have no raw ring.
  pl->sa = 0;
  pl->rs = SK_GRANS;
  if (planes) {
    pl->nb = 3;
    for (uint32_t sa = 8; sa >= 3; --sa)
      if (sk_smem_bytes(d.format, true, pl->bt, sa, pl->nb, pl->rs) <= smem_optin) {
        pl->sa = sa;
        break;
      }
  } else {
    uint32_t sa = (32u * 1024u) / (pl->bt * 128u);
    sa = sa < 3 ? 3 : (sa > 8 ? 8 : sa);
    for (uint32_t nb = 3; nb >= 2 && !pl->sa; --nb)  // (four and five slots measured the same as three)
      for (uint32_t rs = 16; rs >= SK_GRANS && !pl->sa; --rs)
        if (sk_smem_bytes(d.format, false, pl->bt, sa, nb, rs) <= smem_optin) pl->sa = sa, pl->nb = nb, pl->rs = rs;
  }
  if (!pl->sa) return false;
  const uint32_t nk = d.K / SK_UNIT_K;
  pl->per = nk;
  pl->grid = pl->tiles;
  pl->split = false;
  // one CTA per SM, equal runs of units; a run no longer than a tile touches at most two tiles
  if (allow_split && pl->tiles < sm_count) {
    const uint32_t total = pl->tiles * nk;
    uint32_t grid = sm_count < total ? sm_count : total;
    const uint32_t per = (total + grid - 1) / grid;
    grid = (total + per - 1) / per;
    if (per != nk) {
      pl->per = per;
      pl->grid = grid;
      pl->split = true;
    }
  }
  pl->tmem_cols = pl->split ? 512u : 256u;
  pl->cast_bytes = d.a_dtype == CUTB_F32 ? (((uint64_t)d.M * d.K * sizeof(__half) + 15) & ~(uint64_t)15) : 0;
  pl->partial_bytes = pl->split ? (uint64_t)2 * pl->grid * pl->bt * SK_BW * sizeof(float) : 0;
  return true;
}

// The weight as a 2-D tensor of 32-bit words, [N rows][row_bytes / 4]; a box is 256 k of 128 rows.
int make_tmap_w(CUtensorMap *map, const cutb_qmatmul_desc &d) {
  EncodeTiledFn encode = nullptr;
  if (int rc = tc_encode_fn(&encode)) return rc;
  const uint64_t rb = row_bytes(d.format, d.K);
  const cuuint64_t dims[2] = {rb / 4, d.N};
  const cuuint64_t strides[1] = {rb};
  const cuuint32_t box[2] = {sk_row_chunk_bytes(d.format) / 4, SK_GRAN_ROWS};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(d.W), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("qgemm: cuTensorMapEncodeTiled failed with %d for the weight (N=%u row bytes=%llu)", (int)r, d.N,
                   (unsigned long long)rb);
    return CUTB_ERR_CUDA;
  }
  return CUTB_OK;
}

template <int FMT>
int sk_launch(const CUtensorMap &mapA, const CUtensorMap &mapW, const SkParams &p, bool planes, uint32_t grid, bool overlap,
              cudaStream_t stream) {
  static bool configured[64] = {};  // per device: the attribute is set once on each
  int dev = 0;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    DeviceInfo di;
    if (int rc = get_device_info(&di)) return rc;
    CUTB_CUDA_TRY(cudaFuncSetAttribute(qgemm_skinny_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)di.smem_optin));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int fmt = tc_is_plane(FMT) ? CUTB_Q4_0 : FMT;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(sk_threads(FMT));
  cfg.dynamicSmemBytes = sk_smem_bytes(fmt, planes, p.bt, p.sa, p.nb, p.rs);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;
  CUTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, qgemm_skinny_kernel<FMT>, mapA, mapW, p));
  return CUTB_OK;
}

}  // namespace

// Up to 64 tokens always; up to 128 when the prefill kernel's 128-row tiles would leave more than half of the SMs
// idle (there its one-pass epilogue beats this kernel's split and fix-up once the SMs are covered).
bool qgemm_skinny_applies(const cutb_qmatmul_desc &d) {
  if (d.M > 128 || d.K % SK_UNIT_K != 0) return false;
  if (d.M <= 64) return true;
  DeviceInfo di;
  const uint32_t sms = get_device_info(&di) == CUTB_OK ? (uint32_t)di.sm_count : 148u;
  return (d.N + 127) / 128 <= sms / 2;
}

uint64_t qgemm_skinny_workspace(const cutb_qmatmul_desc &d) {
  // fp32 activations are rounded to fp16 rows of K elements first; the stream-K split adds its head / tail slots
  DeviceInfo di;
  uint32_t sms = 148;
  size_t smem = 232448;
  if (get_device_info(&di) == CUTB_OK) sms = (uint32_t)di.sm_count, smem = di.smem_optin;
  SkPlan pl;
  if (!sk_plan(d, sms, smem, true, &pl)) return d.a_dtype == CUTB_F32 ? (uint64_t)d.M * d.K * sizeof(__half) : 0;
  return pl.cast_bytes + pl.partial_bytes;
}

int qgemm_skinny_launch(const cutb_qmatmul_desc &d, cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  SkPlan pl;
  bool ok = sk_plan(d, (uint32_t)di.sm_count, di.smem_optin, true, &pl);
  // without room for the split's slots every tile goes whole to one CTA
  if (ok && pl.split &&
      (!d.workspace || d.workspace_bytes < pl.cast_bytes + pl.partial_bytes || reinterpret_cast<uintptr_t>(d.workspace) % 16 != 0))
    ok = sk_plan(d, (uint32_t)di.sm_count, di.smem_optin, false, &pl);
  if (!ok) {
    set_last_error("qgemm: shared memory too small for the tile rings");
    return CUTB_ERR_UNSUPPORTED;
  }
  SkParams p;
  p.W = reinterpret_cast<const uint8_t *>(d.W);
  p.row_bytes = row_bytes(d.format, d.K);
  p.C = d.C;
  p.ldc = d.ldc;
  p.D = d.D;
  p.ldd = d.ldd;
  p.M = d.M;
  p.K = d.K;
  p.N = d.N;
  p.bt = pl.bt;
  p.sa = pl.sa;
  p.nb = pl.nb;
  p.rs = pl.rs;
  p.tiles = pl.tiles;
  p.per = pl.per;
  p.tmem_cols = pl.tmem_cols;
  p.fusion_type = d.fusion_type;
  p.fusion_op = d.fusion_op;
  p.glu = (d.flags & CUTB_FLAG_GLU_PAIRS) ? 1 : 0;
  p.status = d.status;
  p.partial = nullptr;
  p.vec_ok = reinterpret_cast<uintptr_t>(d.C) % 16 == 0 && d.ldc % 4 == 0 &&
             (d.fusion_type != CUTB_FUSION_BINARY || (reinterpret_cast<uintptr_t>(d.D) % 16 == 0 && d.ldd % 4 == 0));
  p.S = reinterpret_cast<const uint16_t *>(d.scales);
  p.ldb = d.ldb;
  p.lds = d.lds;
  p.blocksK = (d.K + 31) / 32;
  const void *a16 = d.A;
  uint64_t stride = (uint64_t)d.lda * sizeof(__half);
  if (d.a_dtype == CUTB_F32) {
    if (!d.workspace || d.workspace_bytes < pl.cast_bytes || reinterpret_cast<uintptr_t>(d.workspace) % 16 != 0) {
      set_last_error("qgemm: fp32 activations need %llu bytes of 16-byte aligned workspace, got %llu",
                     (unsigned long long)pl.cast_bytes, (unsigned long long)d.workspace_bytes);
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
  if (pl.split) p.partial = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(d.workspace) + pl.cast_bytes);
  CUtensorMap map, mapW;
  if (int rc = make_tmap_a(&map, a16, d.M, d.K, stride, pl.bt)) return rc;
  int rc;
  // after the fp32 cast the activations come from the kernel just before: that launch is the dependency the
  // kernel's griddepcontrol.wait covers, like any other producer of A
  const bool overlap = !(d.flags & CUTB_FLAG_NO_OVERLAP);
  if (d.layout == CUTB_LAYOUT_KN_PLANES) {
    mapW = map;  // unused: the plane converters read global memory themselves
    if (d.format == CUTB_Q8_0) rc = sk_launch<TC_PLANE_Q8>(map, mapW, p, true, pl.grid, overlap, stream);
    else rc = d.affine ? sk_launch<TC_PLANE_Q4A>(map, mapW, p, true, pl.grid, overlap, stream)
                       : sk_launch<TC_PLANE_Q4>(map, mapW, p, true, pl.grid, overlap, stream);
  } else {
    if (int rc2 = make_tmap_w(&mapW, d)) return rc2;
    switch (d.format) {
      case CUTB_Q8_0: rc = sk_launch<CUTB_Q8_0>(map, mapW, p, false, pl.grid, overlap, stream); break;
      case CUTB_Q4_0: rc = sk_launch<CUTB_Q4_0>(map, mapW, p, false, pl.grid, overlap, stream); break;
      default: rc = sk_launch<CUTB_Q4_K>(map, mapW, p, false, pl.grid, overlap, stream); break;
    }
  }
  if (rc != CUTB_OK || !pl.split) return rc;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.tiles, (d.M + SK_FIX_ROWS - 1) / SK_FIX_ROWS);
    cfg.blockDim = dim3(SK_BW);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;  // its predecessor is this library's own kernel
    CUTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, tc_skinny_fixup_kernel, p, d.K / SK_UNIT_K));
  }
  return CUTB_OK;
}

}  // namespace cutb
