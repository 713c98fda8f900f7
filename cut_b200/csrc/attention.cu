// Decode-step attention for one token: rotary embedding of q / k fused with the KV-cache write
// (operators/impl/attention/FusedRoPEKVWrite.cu:13-75) and grouped-query attention of the roped
// query over the populated cache (operators/impl/attention/Attention.cu:31-108).  Position and
// populated length come from a two-word device buffer {pos, seqLen}, as in the reference, so a
// captured step replays for every token.  Cache rows are [position][kv head][head_dim] with a
// row stride padded to 4 elements, elements fp32 or fp16; all arithmetic is fp32.
//
// The reference runs one block per query head, so a KV head is read once per query head of its
// group and at most nHeads blocks are busy.  Here one block owns (KV head, slice of positions):
// every query head of the group is served from one read of the slice.  Two kernels share that plan:
//  * the cluster kernel (head_dim % 32 == 0, 1 / 2 / 4 / 8 query heads per KV head, slices that fit
//    in shared memory -- a 2048-position fp16 cache does): the eight slices of a KV head are one
//    thread-block cluster; K and V rows arrive in shared memory by one wave of async copies and
//    the slices are merged through distributed shared memory, so nothing but the output is written;
//  * the general kernel (any head_dim <= 128, any group size, caches up to 32768 positions): slices
//    read global memory directly, leave partial results in a workspace and are merged by whichever
//    block of the KV head finishes last (an arrival counter; no block waits for another).
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace cutb {
namespace {

constexpr int AT_THREADS = 256;
constexpr int AT_WARPS = AT_THREADS / 32;
constexpr int AT_MAX_HD = 128;     // head_dim limit of the reference kernel (its shared query)
constexpr int AT_MAX_REP = 8;      // query heads per KV head
constexpr int AT_MAX_CHUNK = 512;  // positions per block
constexpr int AT_MAX_SPLITS = 64;
constexpr float AT_NEG = -1e30f;   // the reference's "no score yet"
constexpr int AT_CL = 8;           // blocks per cluster = slices per KV head on the cluster path
constexpr int CL_THREADS = 1024;   // cluster path: one block per SM (shared-memory bound), so fill it with warps
constexpr int CL_WARPS = CL_THREADS / 32;

__device__ __forceinline__ float kv_load(const float *p) { return __ldg(p); }
__device__ __forceinline__ float kv_load(const __half *p) { return __half2float(__ldg(p)); }
__device__ __forceinline__ void kv_store(float *p, float v) { *p = v; }
__device__ __forceinline__ void kv_store(__half *p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ void kv_load4(const float *p, float (&v)[4]) {
  const float4 x = __ldg(reinterpret_cast<const float4 *>(p));
  v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
}
__device__ __forceinline__ void kv_load4(const __half *p, float (&v)[4]) {
  const uint2 x = __ldg(reinterpret_cast<const uint2 *>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&x.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&x.y));
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
}
__device__ __forceinline__ void kv_load2(const float *p, float (&v)[2]) {
  const float2 x = __ldg(reinterpret_cast<const float2 *>(p));
  v[0] = x.x, v[1] = x.y;
}
__device__ __forceinline__ void kv_load2(const __half *p, float (&v)[2]) {
  const uint32_t x = __ldg(reinterpret_cast<const uint32_t *>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&x));
  v[0] = a.x, v[1] = a.y;
}

// One thread per element of q, k and v.  Half-split rotation: element i of the first half of a
// head pairs with element i + head_dim / 2; products and sums are rounded separately (no fused
// multiply-add), so the result is the one plain C arithmetic gives.
template <typename KV>
__global__ void __launch_bounds__(256) rope_kv_write_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                                            const float *__restrict__ v, const uint32_t *__restrict__ params,
                                                            const float *__restrict__ cosT, const float *__restrict__ sinT,
                                                            KV *__restrict__ kC, KV *__restrict__ vC, float *__restrict__ qOut,
                                                            uint32_t qDim, uint32_t kvDim, uint32_t headDim, uint32_t ld,
                                                            uint32_t max_seq, int *status) {
  pdl_enter();
  const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= qDim + 2 * kvDim) return;
  const uint32_t pos = __ldg(params);
  if (pos >= max_seq) {  // never write outside the cache: record it and leave the outputs alone
    if (status && gid == 0) atomicExch(status, (int)CUTB_ERR_INVALID);
    return;
  }
  const uint32_t half = headDim / 2;
  auto rotate = [&](const float *x, uint32_t i) -> float {
    const uint32_t in_head = i % headDim;
    if (in_head < half) {
      const float c = __ldg(cosT + (uint64_t)pos * half + in_head), s = __ldg(sinT + (uint64_t)pos * half + in_head);
      return __fsub_rn(__fmul_rn(__ldg(x + i), c), __fmul_rn(__ldg(x + i + half), s));
    }
    const uint32_t pair = in_head - half;
    const float c = __ldg(cosT + (uint64_t)pos * half + pair), s = __ldg(sinT + (uint64_t)pos * half + pair);
    return __fadd_rn(__fmul_rn(__ldg(x + i - half), s), __fmul_rn(__ldg(x + i), c));
  };
  if (gid < qDim) {
    qOut[gid] = rotate(q, gid);
  } else if (gid < qDim + kvDim) {
    const uint32_t i = gid - qDim;
    kv_store(kC + (uint64_t)pos * ld + i, rotate(k, i));
  } else {
    const uint32_t i = gid - qDim - kvDim;
    kv_store(vC + (uint64_t)pos * ld + i, __ldg(v + i));
  }
}

// Prefill: roped k and v of a batch of tokens into their cache rows (BatchedKVCacheWrite.cu:33-62).
// One block per token; k_in / v_in rows may be columns of a wider matrix (row strides in elements).
template <typename KV>
__global__ void __launch_bounds__(256) batched_kv_write_kernel(const float *__restrict__ kIn, const float *__restrict__ vIn,
                                                               uint32_t kStride, uint32_t vStride, const uint32_t *__restrict__ positions,
                                                               const float *__restrict__ cosT, const float *__restrict__ sinT,
                                                               KV *__restrict__ kC, KV *__restrict__ vC, uint32_t kvDim, uint32_t headDim,
                                                               uint32_t ld, uint32_t max_seq, int *status) {
  pdl_enter();
  const uint32_t token = blockIdx.x, pos = __ldg(positions + token);
  if (pos >= max_seq) {
    if (status && threadIdx.x == 0) atomicExch(status, (int)CUTB_ERR_INVALID);
    return;
  }
  const uint32_t half = headDim / 2;
  const float *k = kIn + (uint64_t)token * kStride, *v = vIn + (uint64_t)token * vStride;
  const float *cs = cosT + (uint64_t)pos * half, *sn = sinT + (uint64_t)pos * half;
  for (uint32_t i = threadIdx.x; i < kvDim; i += blockDim.x) {
    const uint32_t in_head = i % headDim;
    const float kr = in_head < half ? __fsub_rn(__fmul_rn(__ldg(k + i), __ldg(cs + in_head)), __fmul_rn(__ldg(k + i + half), __ldg(sn + in_head)))
                                    : __fadd_rn(__fmul_rn(__ldg(k + i - half), __ldg(sn + in_head - half)), __fmul_rn(__ldg(k + i), __ldg(cs + in_head - half)));
    kv_store(kC + (uint64_t)pos * ld + i, kr);
    kv_store(vC + (uint64_t)pos * ld + i, __ldg(v + i));
  }
}

struct AttnParams {
  const float *q;
  const void *kC, *vC;
  const uint32_t *params;
  float *out;
  float *part_acc;  // [nHeads][splits][headDim]
  float *part_m;    // [nHeads][splits]
  float *part_l;    // [nHeads][splits]
  unsigned int *counters;  // [nKvHeads], zero between launches
  int *status;
  uint32_t nHeads, nKvHeads, headDim, ld, nRep, max_seq, splits;
  uint32_t chunk_cap;  // cluster path: rows a block's shared-memory tiles hold
  // fused RoPE + cache write (cluster path; k_new == nullptr: plain attention): q is the unrotated query
  const float *k_new, *v_new, *cosT, *sinT;
  // batched (prefill) mode of the general kernel: one block per (KV head, token); token i attends rows [0, positions[i]]
  // with its query rotated here; q and out advance by their strides per token
  const uint32_t *positions;
  uint32_t q_stride, out_stride;
  uint32_t tq, n_tokens;  // batched mode: consecutive tokens served by one block (they share every K / V row it reads)
  float scale;
};

// grid = (nKvHeads, splits).  VEC: head_dim % 32 == 0 and 16-byte aligned rows, so eight lanes
// cover one position with 4-element loads; otherwise the same plan with scalar loads.
template <typename KV, bool VEC>
__global__ void __launch_bounds__(AT_THREADS) attention_decode_kernel(const AttnParams p) {
  __shared__ __align__(16) float qs[AT_MAX_REP * AT_MAX_HD];
  __shared__ float sc[AT_MAX_REP * AT_MAX_CHUNK];
  __shared__ __align__(16) float red[AT_MAX_REP * 2 * AT_THREADS];
  __shared__ float head_m[AT_MAX_REP], head_l[AT_MAX_REP];
  __shared__ float wts[AT_MAX_REP * AT_MAX_SPLITS];
  __shared__ int is_last;

  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t kvH = blockIdx.x, split = blockIdx.y, S = p.splits;
  const uint32_t HD = p.headDim;
  const bool batched = p.positions != nullptr;
  // Batched mode: a block serves TQ consecutive tokens.  Their query heads are "virtual heads" of the KV head
  // (token-major), each with its own populated length; below, nRep counts virtual heads.
  const uint32_t realRep = p.nRep, TQ = batched ? p.tq : 1u, nRep = realRep * TQ;
  const uint32_t token0 = batched ? blockIdx.z * TQ : 0u;
  __shared__ uint32_t vseq[AT_MAX_REP];  // rows [0, vseq) attended by each virtual head
  pdl_enter();
  const uint32_t seq_cap = p.max_seq;  // (a batched block walks its whole range in chunks of AT_MAX_CHUNK rows)
  uint32_t seqLen = 0;
  if (batched) {
    for (uint32_t tq = 0; tq < TQ; ++tq) {
      uint32_t sl = token0 + tq < p.n_tokens ? __ldg(p.positions + token0 + tq) + 1u : 0u;
      if (sl > seq_cap) {  // never read outside the cache (or past what one block holds)
        if (p.status && tid == 0 && kvH == 0) atomicExch(p.status, (int)CUTB_ERR_INVALID);
        sl = seq_cap;
      }
      if (tid < realRep) vseq[tq * realRep + tid] = sl;
      seqLen = max(seqLen, sl);
    }
  } else {
    seqLen = __ldg(p.params + 1);
    if (seqLen > seq_cap) {
      if (p.status && tid == 0 && kvH == 0 && split == 0) atomicExch(p.status, (int)CUTB_ERR_INVALID);
      seqLen = seq_cap;
    }
  }
  // Decode mode: this block's slice [t0, t1) of the range, at most AT_MAX_CHUNK rows by the launcher's choice of S,
  // one pass.  Batched mode (S = 1): the block walks [0, seqLen) in chunks of AT_MAX_CHUNK rows with a running
  // maximum and exp-sum per virtual head; the weighted V sums in registers are rescaled when the maximum moves.
  const uint32_t chunk = batched ? (uint32_t)AT_MAX_CHUNK : (seqLen + S - 1) / S;
  const uint32_t nchunks = batched ? max(1u, (seqLen + chunk - 1) / chunk) : 1u;
  __shared__ float run_fac[AT_MAX_REP];
  if (tid < AT_MAX_REP) head_m[tid] = AT_NEG, head_l[tid] = 0.f;
  const KV *kC = reinterpret_cast<const KV *>(p.kC) + (uint64_t)kvH * HD;
  const KV *vC = reinterpret_cast<const KV *>(p.vC) + (uint64_t)kvH * HD;

  if (batched) {  // rotate every token's query heads at its own position (half-split, separately rounded products)
    const uint32_t half = HD / 2;
    for (uint32_t i = tid; i < nRep * HD; i += AT_THREADS) {
      const uint32_t vr = i / HD, in_head = i % HD, tq = vr / realRep, r = vr % realRep, tk = token0 + tq;
      float val = 0.f;
      if (tk < p.n_tokens) {
        const uint32_t pos = min(__ldg(p.positions + tk), seq_cap - 1);
        const float *x = p.q + (uint64_t)tk * p.q_stride + (uint64_t)(kvH * realRep + r) * HD + in_head;
        const float *cs = p.cosT + (uint64_t)pos * half, *sn = p.sinT + (uint64_t)pos * half;
        val = in_head < half ? __fsub_rn(__fmul_rn(__ldg(x), __ldg(cs + in_head)), __fmul_rn(__ldg(x + half), __ldg(sn + in_head)))
                             : __fadd_rn(__fmul_rn(__ldg(x - half), __ldg(sn + in_head - half)), __fmul_rn(__ldg(x), __ldg(cs + in_head - half)));
      }
      qs[i] = val;
    }
  } else {
    for (uint32_t i = tid; i < nRep * HD; i += AT_THREADS) qs[i] = __ldg(p.q + (uint64_t)kvH * nRep * HD + i);
  }
  __syncthreads();

  constexpr uint32_t EV = VEC ? 2 : 1;
  float acc[AT_MAX_REP][EV];
#pragma unroll
  for (int r = 0; r < AT_MAX_REP; ++r)
#pragma unroll
    for (uint32_t e = 0; e < EV; ++e) acc[r][e] = 0.f;
  uint32_t t0 = 0, t1 = 0, cnt = 0;
  for (uint32_t ci = 0; ci < nchunks; ++ci) {
  t0 = min((batched ? ci : split) * chunk, seqLen), t1 = min(t0 + chunk, seqLen), cnt = t1 - t0;
  // scores: eight lanes per position, four positions per warp and pass; the loads of up to four
  // passes are issued before the first is used, so a slice costs one or two memory round trips
  {
    const uint32_t j = lane & 7, sub = lane >> 3;
    constexpr uint32_t PU = 4;                 // passes in flight
    constexpr uint32_t STEP = AT_WARPS * 4;    // positions per pass of the block
    for (uint32_t tb = t0 + warp * 4; tb < t1; tb += STEP * PU) {
      if constexpr (VEC) {
        float kv[PU][AT_MAX_HD / 32][4];
#pragma unroll
        for (uint32_t u = 0; u < PU; ++u) {
          const uint32_t t = tb + u * STEP + sub;
          const KV *kp = kC + (uint64_t)t * p.ld;
#pragma unroll
          for (uint32_t i = 0; i < AT_MAX_HD / 32; ++i) {
            const uint32_t e = 4 * j + 32 * i;
            if (t < t1 && e < HD) kv_load4(kp + e, kv[u][i]);
            else kv[u][i][0] = kv[u][i][1] = kv[u][i][2] = kv[u][i][3] = 0.f;
          }
        }
#pragma unroll
        for (uint32_t u = 0; u < PU; ++u) {
          const uint32_t t = tb + u * STEP + sub;
          if (tb + u * STEP >= t1) break;  // warp-uniform
          float dot[AT_MAX_REP];
#pragma unroll
          for (int r = 0; r < AT_MAX_REP; ++r) dot[r] = 0.f;
#pragma unroll
          for (uint32_t i = 0; i < AT_MAX_HD / 32; ++i) {
            const uint32_t e = 4 * j + 32 * i;
            if (e < HD) {
#pragma unroll
              for (int r = 0; r < AT_MAX_REP; ++r)
                if (r < nRep) {
                  const float4 qv = *reinterpret_cast<const float4 *>(&qs[r * HD + e]);
                  dot[r] = fmaf(qv.x, kv[u][i][0], fmaf(qv.y, kv[u][i][1], fmaf(qv.z, kv[u][i][2], fmaf(qv.w, kv[u][i][3], dot[r]))));
                }
            }
          }
#pragma unroll
          for (int r = 0; r < AT_MAX_REP; ++r)
            if (r < nRep) {
              float d = dot[r];
              d += __shfl_xor_sync(0xffffffffu, d, 1);
              d += __shfl_xor_sync(0xffffffffu, d, 2);
              d += __shfl_xor_sync(0xffffffffu, d, 4);
              if (t < t1 && j == 0) sc[r * AT_MAX_CHUNK + (t - t0)] = d * p.scale;
            }
        }
      } else {
        for (uint32_t u = 0; u < PU; ++u) {
          const uint32_t t = tb + u * STEP + sub;
          if (tb + u * STEP >= t1) break;  // warp-uniform
          float dot[AT_MAX_REP];
#pragma unroll
          for (int r = 0; r < AT_MAX_REP; ++r) dot[r] = 0.f;
          if (t < t1) {
            const KV *kp = kC + (uint64_t)t * p.ld;
            for (uint32_t e = j; e < HD; e += 8) {
              const float kvv = kv_load(kp + e);
#pragma unroll
              for (int r = 0; r < AT_MAX_REP; ++r)
                if (r < nRep) dot[r] = fmaf(qs[r * HD + e], kvv, dot[r]);
            }
          }
#pragma unroll
          for (int r = 0; r < AT_MAX_REP; ++r)
            if (r < nRep) {
              float d = dot[r];
              d += __shfl_xor_sync(0xffffffffu, d, 1);
              d += __shfl_xor_sync(0xffffffffu, d, 2);
              d += __shfl_xor_sync(0xffffffffu, d, 4);
              if (t < t1 && j == 0) sc[r * AT_MAX_CHUNK + (t - t0)] = d * p.scale;
            }
        }
      }
    }
  }
  __syncthreads();

  // slice softmax: warp r owns query head r of the group
  for (uint32_t r = warp; r < nRep; r += AT_WARPS) {
    // a token of the tile sees the rows up to its own only
    const uint32_t cr = batched ? (vseq[r] > t0 ? min(vseq[r] - t0, cnt) : 0u) : cnt;
    float m = head_m[r];  // the maximum so far (AT_NEG before the first chunk)
    for (uint32_t i = lane; i < cr; i += 32) m = fmaxf(m, sc[r * AT_MAX_CHUNK + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float fac = expf(head_m[r] - m);  // 1 while the maximum stands (and for the only chunk of the decode mode)
    float l = 0.f;
    for (uint32_t i = lane; i < cr; i += 32) {
      const float e = expf(sc[r * AT_MAX_CHUNK + i] - m);
      sc[r * AT_MAX_CHUNK + i] = e;
      l += e;
    }
    for (uint32_t i = cr + lane; i < cnt; i += 32) sc[r * AT_MAX_CHUNK + i] = 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    __syncwarp();
    if (lane == 0) run_fac[r] = fac, head_l[r] = fmaf(head_l[r], fac, l), head_m[r] = m;
  }
  __syncthreads();

  // weighted V sum: thread (tg, tp) adds positions tg, tg + G, ... for EV dimensions of every head
  {
    const uint32_t P = HD / EV, G = AT_THREADS / P;
    const uint32_t tp = tid % P, tg = tid / P;
    if (nchunks > 1) {
#pragma unroll
      for (int r = 0; r < AT_MAX_REP; ++r)
        if (r < nRep) {
#pragma unroll
          for (uint32_t e = 0; e < EV; ++e) acc[r][e] *= run_fac[r];
        }
    }
    if (tg < G) {
      constexpr uint32_t VU = 8;  // rows in flight per thread
      for (uint32_t ib = tg; ib < cnt; ib += G * VU) {
        float vv[VU][EV];
#pragma unroll
        for (uint32_t u = 0; u < VU; ++u) {
          const uint32_t i = ib + u * G;
          const KV *vp = vC + (uint64_t)(t0 + i) * p.ld + tp * EV;
          if (i < cnt) {
            if constexpr (VEC) kv_load2(vp, vv[u]);
            else vv[u][0] = kv_load(vp);
          } else {
#pragma unroll
            for (uint32_t e = 0; e < EV; ++e) vv[u][e] = 0.f;
          }
        }
#pragma unroll
        for (uint32_t u = 0; u < VU; ++u) {
          const uint32_t i = ib + u * G;
          if (i < cnt) {
#pragma unroll
            for (int r = 0; r < AT_MAX_REP; ++r)
              if (r < nRep) {
                const float w = sc[r * AT_MAX_CHUNK + i];
#pragma unroll
                for (uint32_t e = 0; e < EV; ++e) acc[r][e] = fmaf(w, vv[u][e], acc[r][e]);
              }
          }
        }
      }
    }
  }
  __syncthreads();  // the next chunk overwrites the scores
  }  // chunks

  {
    const uint32_t P = HD / EV, G = AT_THREADS / P;
    const uint32_t tp = tid % P, tg = tid / P;
    if (tg < G) {
#pragma unroll
      for (int r = 0; r < AT_MAX_REP; ++r)
        if (r < nRep) {
#pragma unroll
          for (uint32_t e = 0; e < EV; ++e) red[(tg * nRep + r) * HD + tp * EV + e] = acc[r][e];
        }
    }
    __syncthreads();
    if (S == 1) {  // one slice: it is the result (an empty range gives zeros, as the reference's sum does)
      for (uint32_t idx = tid; idx < nRep * HD; idx += AT_THREADS) {
        const uint32_t r = idx / HD, d = idx % HD;
        float s = 0.f;
        for (uint32_t g = 0; g < G; ++g) s += red[(g * nRep + r) * HD + d];
        const uint32_t tk = token0 + r / realRep;
        if (!batched || tk < p.n_tokens)
          p.out[(uint64_t)tk * p.out_stride + (uint64_t)(kvH * realRep + r % realRep) * HD + d] = head_l[r] > 0.f ? s / head_l[r] : 0.f;
      }
      return;
    }
    for (uint32_t idx = tid; idx < nRep * HD; idx += AT_THREADS) {
      const uint32_t r = idx / HD, d = idx % HD;
      float s = 0.f;
      for (uint32_t g = 0; g < G; ++g) s += red[(g * nRep + r) * HD + d];
      p.part_acc[((uint64_t)(kvH * nRep + r) * S + split) * HD + d] = s;
    }
    if (tid < nRep) {
      p.part_m[(kvH * nRep + tid) * S + split] = head_m[tid];
      p.part_l[(kvH * nRep + tid) * S + split] = head_l[tid];
    }
  }

  // the block that arrives last for this KV head merges the slices; nobody waits
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int prev = atomicAdd(p.counters + kvH, 1u);
    is_last = prev == S - 1;
    if (is_last) p.counters[kvH] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (uint32_t r = warp; r < nRep; r += AT_WARPS) {
    const uint32_t h = kvH * nRep + r;
    float m = AT_NEG;
    for (uint32_t s = lane; s < S; s += 32) m = fmaxf(m, __ldcg(p.part_m + h * S + s));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.f;
    for (uint32_t s = lane; s < S; s += 32) {
      const float w = expf(__ldcg(p.part_m + h * S + s) - m);
      wts[r * AT_MAX_SPLITS + s] = w;
      l = fmaf(w, __ldcg(p.part_l + h * S + s), l);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) head_l[r] = l > 0.f ? 1.f / l : 0.f;  // an empty cache gives zeros, as the reference's sum does
  }
  __syncthreads();
  for (uint32_t idx = tid; idx < nRep * HD; idx += AT_THREADS) {
    const uint32_t r = idx / HD, d = idx % HD, h = kvH * nRep + r;
    float s = 0.f;
    for (uint32_t sb = 0; sb < S; sb += 8) {  // eight loads in flight
      float a[8];
#pragma unroll
      for (uint32_t u = 0; u < 8; ++u) a[u] = sb + u < S ? __ldcg(p.part_acc + ((uint64_t)h * S + sb + u) * HD + d) : 0.f;
#pragma unroll
      for (uint32_t u = 0; u < 8; ++u)
        if (sb + u < S) s = fmaf(wts[r * AT_MAX_SPLITS + sb + u], a[u], s);
    }
    p.out[(uint64_t)h * HD + d] = s * head_l[r];
  }
}

// Cluster path (caches whose slices fit in shared memory; head_dim % 32 == 0): the slices of one
// KV head are the blocks of one thread-block cluster.  Each block brings its K and V rows into
// shared memory with one wave of 16-byte async copies (one memory round trip for both), works
// from there, and the slices are merged through distributed shared memory: after a cluster
// barrier every block reads all blocks' maxima, exp-sums and partial outputs for its share of
// the output.  No partial result touches global memory.  grid = (nKvHeads, S), cluster (1, S, 1).
__device__ __forceinline__ void smem_load4(const float *p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4 *>(p);
  v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
}
__device__ __forceinline__ void smem_load4(const __half *p, float (&v)[4]) {
  const uint2 x = *reinterpret_cast<const uint2 *>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&x.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&x.y));
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
}
__device__ __forceinline__ float2 smem_load2(const float *p) { return *reinterpret_cast<const float2 *>(p); }
__device__ __forceinline__ float2 smem_load2(const __half *p) { return __half22float2(*reinterpret_cast<const __half2 *>(p)); }

template <typename KV, int NREP>
__global__ void __launch_bounds__(CL_THREADS) attention_decode_cluster_kernel(const AttnParams p) {
  extern __shared__ __align__(16) uint8_t tiles[];  // K rows, V rows (row stride RS bytes), then the V-sum scratch
  __shared__ __align__(16) float qs[NREP * AT_MAX_HD];
  __shared__ float sc[NREP * AT_MAX_CHUNK];
  __shared__ float pacc[NREP * AT_MAX_HD];
  __shared__ float head_m[NREP], head_l[NREP];

  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t kvH = blockIdx.x, split = blockIdx.y, S = gridDim.y;
  constexpr uint32_t nRep = NREP;
  const uint32_t HD = p.headDim;
  pdl_enter();
  uint32_t seqLen = __ldg(p.params + 1);
  if (seqLen > p.max_seq) {
    if (p.status && tid == 0 && kvH == 0 && split == 0) atomicExch(p.status, (int)CUTB_ERR_INVALID);
    seqLen = p.max_seq;
  }
  const uint32_t chunk = (seqLen + S - 1) / S;  // <= chunk_cap
  const uint32_t t0 = min(split * chunk, seqLen), t1 = min(t0 + chunk, seqLen), cnt = t1 - t0;
  const uint32_t row_bytes = HD * (uint32_t)sizeof(KV), RS = row_bytes + 16;  // padded: rows start on different banks
  // fused mode: this token's K / V row is rotated here, put into the slice that owns its position and
  // written to the cache by the first slice; the copies below never touch that row
  const bool fused = p.k_new != nullptr;
  uint32_t pos = 0xFFFFFFFFu;
  if (fused) {
    pos = __ldg(p.params);
    if (pos >= p.max_seq) {  // never write outside the cache: record it, rotate nothing
      if (p.status && tid == 0 && kvH == 0 && split == 0) atomicExch(p.status, (int)CUTB_ERR_INVALID);
      pos = 0xFFFFFFFFu;
    }
  }
  const bool own = pos >= t0 && pos < t1;
  uint8_t *ktile = tiles, *vtile = tiles + (size_t)p.chunk_cap * RS;
  float *red = reinterpret_cast<float *>(tiles + (size_t)2 * p.chunk_cap * RS);  // [G][NREP][HD]
  {
    const uint32_t ppr = row_bytes / 16, total = cnt * ppr;
    const uint8_t *kg = reinterpret_cast<const uint8_t *>(p.kC) + ((uint64_t)t0 * p.ld + (uint64_t)kvH * HD) * sizeof(KV);
    const uint8_t *vg = reinterpret_cast<const uint8_t *>(p.vC) + ((uint64_t)t0 * p.ld + (uint64_t)kvH * HD) * sizeof(KV);
    const uint64_t gstride = (uint64_t)p.ld * sizeof(KV);
    for (uint32_t id = tid; id < total; id += CL_THREADS) {
      const uint32_t r = id / ppr, c = id % ppr;
      if (own && r == pos - t0) continue;
      const uint32_t kd = (uint32_t)__cvta_generic_to_shared(ktile + (size_t)r * RS + c * 16);
      const uint32_t vd = (uint32_t)__cvta_generic_to_shared(vtile + (size_t)r * RS + c * 16);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kd), "l"(kg + r * gstride + c * 16) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vd), "l"(vg + r * gstride + c * 16) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  if (pos != 0xFFFFFFFFu) {
    const uint32_t half = HD / 2;
    const float *cs = p.cosT + (uint64_t)pos * half, *sn = p.sinT + (uint64_t)pos * half;
    // half-split rotation with separately rounded products, as the stand-alone kernel computes it
    auto rotate = [&](const float *x, uint32_t i) -> float {
      const uint32_t in_head = i % HD;
      if (in_head < half) return __fsub_rn(__fmul_rn(__ldg(x + i), __ldg(cs + in_head)), __fmul_rn(__ldg(x + i + half), __ldg(sn + in_head)));
      return __fadd_rn(__fmul_rn(__ldg(x + i - half), __ldg(sn + in_head - half)), __fmul_rn(__ldg(x + i), __ldg(cs + in_head - half)));
    };
    for (uint32_t i = tid; i < nRep * HD; i += CL_THREADS) qs[i] = rotate(p.q + (uint64_t)kvH * nRep * HD, i);
    if (own || split == 0) {
      for (uint32_t e = tid; e < HD; e += CL_THREADS) {
        const float kr = rotate(p.k_new + (uint64_t)kvH * HD, e), vv = __ldg(p.v_new + (uint64_t)kvH * HD + e);
        if (own) {
          kv_store(reinterpret_cast<KV *>(ktile + (size_t)(pos - t0) * RS) + e, kr);
          kv_store(reinterpret_cast<KV *>(vtile + (size_t)(pos - t0) * RS) + e, vv);
        }
        if (split == 0) {
          const uint64_t at = (uint64_t)pos * p.ld + (uint64_t)kvH * HD + e;
          kv_store(reinterpret_cast<KV *>(const_cast<void *>(p.kC)) + at, kr);
          kv_store(reinterpret_cast<KV *>(const_cast<void *>(p.vC)) + at, vv);
        }
      }
    }
  } else {
    for (uint32_t i = tid; i < nRep * HD; i += CL_THREADS) qs[i] = __ldg(p.q + (uint64_t)kvH * nRep * HD + i);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  {  // scores: eight lanes per row, four rows per warp and pass
    const uint32_t j = lane & 7, sub = lane >> 3;
    for (uint32_t ib = warp * 4; ib < cnt; ib += CL_WARPS * 4) {
      const uint32_t i = ib + sub;
      const bool valid = i < cnt;
      float dot[NREP];
#pragma unroll
      for (int r = 0; r < NREP; ++r) dot[r] = 0.f;
      if (valid) {
        const KV *kp = reinterpret_cast<const KV *>(ktile + (size_t)i * RS);
        for (uint32_t e = 4 * j; e < HD; e += 32) {
          float kv[4];
          smem_load4(kp + e, kv);
#pragma unroll
          for (int r = 0; r < NREP; ++r)
            {
              const float4 qv = *reinterpret_cast<const float4 *>(&qs[r * HD + e]);
              dot[r] = fmaf(qv.x, kv[0], fmaf(qv.y, kv[1], fmaf(qv.z, kv[2], fmaf(qv.w, kv[3], dot[r]))));
            }
        }
      }
#pragma unroll
      for (int r = 0; r < NREP; ++r)
        {
          float d = dot[r];
          d += __shfl_xor_sync(0xffffffffu, d, 1);
          d += __shfl_xor_sync(0xffffffffu, d, 2);
          d += __shfl_xor_sync(0xffffffffu, d, 4);
          if (valid && j == 0) sc[r * AT_MAX_CHUNK + i] = d * p.scale;
        }
    }
  }
  __syncthreads();

  for (uint32_t r = warp; r < nRep; r += CL_WARPS) {  // slice softmax: warp r owns query head r of the group
    float m = AT_NEG;
    for (uint32_t i = lane; i < cnt; i += 32) m = fmaxf(m, sc[r * AT_MAX_CHUNK + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.f;
    for (uint32_t i = lane; i < cnt; i += 32) {
      const float e = expf(sc[r * AT_MAX_CHUNK + i] - m);
      sc[r * AT_MAX_CHUNK + i] = e;
      l += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) head_m[r] = m, head_l[r] = l;
  }
  __syncthreads();

  {  // weighted V sum: thread (tg, tp) adds rows tg, tg + G, ... for two dimensions of every head
    const uint32_t P = HD / 2, G = CL_THREADS / P;
    const uint32_t tp = tid % P, tg = tid / P;
    float acc[NREP][2];
#pragma unroll
    for (int r = 0; r < NREP; ++r) acc[r][0] = acc[r][1] = 0.f;
    if (tg < G) {
      for (uint32_t i = tg; i < cnt; i += G) {
        const float2 vv = smem_load2(reinterpret_cast<const KV *>(vtile + (size_t)i * RS) + 2 * tp);
#pragma unroll
        for (int r = 0; r < NREP; ++r)
          {
            const float w = sc[r * AT_MAX_CHUNK + i];
            acc[r][0] = fmaf(w, vv.x, acc[r][0]);
            acc[r][1] = fmaf(w, vv.y, acc[r][1]);
          }
      }
#pragma unroll
      for (int r = 0; r < NREP; ++r)
        *reinterpret_cast<float2 *>(&red[(tg * nRep + r) * HD + 2 * tp]) = make_float2(acc[r][0], acc[r][1]);
    }
    __syncthreads();
    for (uint32_t idx = tid; idx < nRep * HD; idx += CL_THREADS) {
      const uint32_t r = idx / HD, d = idx % HD;
      float s = 0.f;
      for (uint32_t g = 0; g < G; ++g) s += red[(g * nRep + r) * HD + d];
      pacc[idx] = s;
    }
  }
  cluster.sync();  // every block's pacc / head_m / head_l are in place

  {  // merge: block `split` finishes its share of the nRep * HD outputs of this KV head
    const uint32_t tot = nRep * HD, per = (tot + S - 1) / S, idx = split * per + tid;
    if (tid < per && idx < tot) {
      const uint32_t r = idx / HD;
      float m_s[AT_CL], l_s[AT_CL], a_s[AT_CL];
#pragma unroll
      for (uint32_t s2 = 0; s2 < AT_CL; ++s2) {
        if (s2 < S) {
          m_s[s2] = cluster.map_shared_rank(head_m, s2)[r];
          l_s[s2] = cluster.map_shared_rank(head_l, s2)[r];
          a_s[s2] = cluster.map_shared_rank(pacc, s2)[idx];
        } else {
          m_s[s2] = AT_NEG, l_s[s2] = 0.f, a_s[s2] = 0.f;
        }
      }
      float m = AT_NEG;
#pragma unroll
      for (uint32_t s2 = 0; s2 < AT_CL; ++s2) m = fmaxf(m, m_s[s2]);
      float l = 0.f, a = 0.f;
#pragma unroll
      for (uint32_t s2 = 0; s2 < AT_CL; ++s2) {
        const float w = expf(m_s[s2] - m);
        l = fmaf(w, l_s[s2], l);
        a = fmaf(w, a_s[s2], a);
      }
      p.out[(uint64_t)kvH * tot + idx] = l > 0.f ? a / l : 0.f;  // an empty cache gives zeros, as the reference's sum does
    }
  }
  cluster.sync();  // nobody leaves while its shared memory may still be read
}

constexpr size_t AT_CLUSTER_SMEM = 200 * 1024;  // dynamic shared memory the cluster path may ask for (beside <= 25 KB static)

template <typename KV, int NREP>
int cluster_launch(const AttnParams &p, uint32_t S, size_t dyn, cudaStream_t stream) {
  static bool configured[64] = {};  // per device: the attribute is set once on each
  int dev = 0;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    CUTB_CUDA_TRY(cudaFuncSetAttribute(attention_decode_cluster_kernel<KV, NREP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)AT_CLUSTER_SMEM));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.nKvHeads, S);
  cfg.blockDim = dim3(CL_THREADS);
  cfg.dynamicSmemBytes = dyn;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = S;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  CUTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, attention_decode_cluster_kernel<KV, NREP>, p));
  return CUTB_OK;
}

// SM count of the current device; 148 (a B200) only when no device can be queried, so that sizes can
// be computed ahead of time on a host without one.
uint32_t sm_count_or_default() {
  DeviceInfo di;
  return (get_device_info(&di) == CUTB_OK && di.sm_count > 0) ? (uint32_t)di.sm_count : 148u;
}

// The kernels index cache rows with 32-bit strides.
int check_ld(uint64_t ld, const char *who) {
  if (ld > 0xFFFFFFFFull) {
    set_last_error("%s: row stride %llu does not fit 32 bits", who, (unsigned long long)ld);
    return CUTB_ERR_INVALID;
  }
  return CUTB_OK;
}

uint32_t attn_splits(uint32_t nKvHeads, uint32_t max_seq) {
  uint32_t s = sm_count_or_default() / nKvHeads;
  if (s < 1) s = 1;
  if (s > (uint32_t)AT_MAX_SPLITS) s = AT_MAX_SPLITS;
  if (s > max_seq) s = max_seq;
  while (s < (uint32_t)AT_MAX_SPLITS && (max_seq + s - 1) / s > (uint32_t)AT_MAX_CHUNK) ++s;
  return s;
}

}  // namespace

int rope_kv_write_launch(int kv_dtype, const float *q, const float *k, const float *v, const uint32_t *params, const float *cosT,
                         const float *sinT, void *kC, void *vC, float *qOut, uint32_t qDim, uint32_t kvDim, uint32_t headDim,
                         uint64_t ld, uint32_t max_seq, int *status, cudaStream_t stream) {
  if (int rc = check_ld(ld, "rope_kv_write_launch")) return rc;
  const uint32_t total = qDim + 2 * kvDim;
  const dim3 grid((total + 255) / 256);
  if (kv_dtype == CUTB_F16)
    CUTB_CUDA_TRY(launch_pdl(rope_kv_write_kernel<__half>, grid, dim3(256), 0, stream, q, k, v, params, cosT, sinT, (__half *)kC,
                             (__half *)vC, qOut, qDim, kvDim, headDim, (uint32_t)ld, max_seq, status));
  else
    CUTB_CUDA_TRY(launch_pdl(rope_kv_write_kernel<float>, grid, dim3(256), 0, stream, q, k, v, params, cosT, sinT, (float *)kC,
                             (float *)vC, qOut, qDim, kvDim, headDim, (uint32_t)ld, max_seq, status));
  return CUTB_OK;
}

// Workspace: 256 bytes of arrival counters (zero before the first launch; every launch leaves
// them zero), then the slices' partial sums, maxima and exp-sums, then one rotated query (used
// when a fused request runs as two launches).
uint64_t attention_workspace_bytes(uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint32_t max_seq) {
  if (nKvHeads == 0 || max_seq == 0) return 0;
  const uint64_t S = attn_splits(nKvHeads, max_seq);
  return 256 + (uint64_t)nHeads * S * (headDim + 2) * sizeof(float) + (uint64_t)nHeads * headDim * sizeof(float);
}

namespace {
// Plain attention (k_new == nullptr) or RoPE + cache write + attention in one launch where the cluster kernel applies;
// elsewhere the fused request runs as the stand-alone rotation kernel followed by the general attention kernel.
int attention_launch_any(int kv_dtype, const float *q, const float *k_new, const float *v_new, const float *cosT, const float *sinT,
                         void *kC, void *vC, const uint32_t *params, float *out, uint32_t nHeads, uint32_t nKvHeads,
                         uint32_t headDim, uint64_t ld, uint32_t max_seq, float scale, void *workspace, int *status,
                         cudaStream_t stream) {
  AttnParams p{};
  p.k_new = k_new, p.v_new = v_new, p.cosT = cosT, p.sinT = sinT;
  p.q = q, p.kC = kC, p.vC = vC, p.params = params, p.out = out, p.status = status;
  p.nHeads = nHeads, p.nKvHeads = nKvHeads, p.headDim = headDim, p.ld = (uint32_t)ld, p.nRep = nHeads / nKvHeads;
  p.max_seq = max_seq, p.scale = scale;
  p.splits = attn_splits(nKvHeads, max_seq);
  if ((max_seq + p.splits - 1) / p.splits > (uint32_t)AT_MAX_CHUNK) {
    set_last_error("attention: cache longer than 32768 positions");
    return CUTB_ERR_UNSUPPORTED;
  }
  p.counters = reinterpret_cast<unsigned int *>(workspace);
  p.part_acc = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(workspace) + 256);
  p.part_m = p.part_acc + (uint64_t)nHeads * p.splits * headDim;
  p.part_l = p.part_m + (uint64_t)nHeads * p.splits;
  const uint32_t esz = kv_dtype == CUTB_F16 ? 2 : 4;
  const bool vec = headDim % 32 == 0 && (ld * esz) % 16 == 0 && reinterpret_cast<uintptr_t>(kC) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(vC) % 16 == 0;
  // cluster path: eight slices per KV head (fewer for tiny caches), K and V slices in shared memory
  {
    const uint32_t S = max_seq < (uint32_t)AT_CL ? max_seq : (uint32_t)AT_CL;
    const uint32_t cap = (max_seq + S - 1) / S;
    const uint32_t groups = CL_THREADS / (headDim / 2 ? headDim / 2 : 1);
    const size_t dyn = (size_t)2 * cap * (headDim * esz + 16) + (size_t)groups * p.nRep * headDim * sizeof(float);
    const bool rep_ok = p.nRep == 1 || p.nRep == 2 || p.nRep == 4 || p.nRep == 8;
    if (vec && rep_ok && cap <= (uint32_t)AT_MAX_CHUNK && dyn <= AT_CLUSTER_SMEM) {
      p.splits = S;
      p.chunk_cap = cap;
      const bool h = kv_dtype == CUTB_F16;
      switch (p.nRep) {
        case 1: return h ? cluster_launch<__half, 1>(p, S, dyn, stream) : cluster_launch<float, 1>(p, S, dyn, stream);
        case 2: return h ? cluster_launch<__half, 2>(p, S, dyn, stream) : cluster_launch<float, 2>(p, S, dyn, stream);
        case 4: return h ? cluster_launch<__half, 4>(p, S, dyn, stream) : cluster_launch<float, 4>(p, S, dyn, stream);
        default: return h ? cluster_launch<__half, 8>(p, S, dyn, stream) : cluster_launch<float, 8>(p, S, dyn, stream);
      }
    }
  }
  if (k_new) {  // not fusable here: rotate into the scratch behind the partial sums, then attend
    float *q_roped = p.part_l + (uint64_t)nHeads * p.splits;
    if (int rc = rope_kv_write_launch(kv_dtype, q, k_new, v_new, params, cosT, sinT, kC, vC, q_roped, nHeads * headDim,
                                      nKvHeads * headDim, headDim, ld, max_seq, status, stream))
      return rc;
    p.q = q_roped;
    p.k_new = p.v_new = p.cosT = p.sinT = nullptr;
  }
  const dim3 grid(nKvHeads, p.splits);
  if (kv_dtype == CUTB_F16) {
    if (vec) CUTB_CUDA_TRY(launch_pdl(attention_decode_kernel<__half, true>, grid, dim3(AT_THREADS), 0, stream, p));
    else CUTB_CUDA_TRY(launch_pdl(attention_decode_kernel<__half, false>, grid, dim3(AT_THREADS), 0, stream, p));
  } else {
    if (vec) CUTB_CUDA_TRY(launch_pdl(attention_decode_kernel<float, true>, grid, dim3(AT_THREADS), 0, stream, p));
    else CUTB_CUDA_TRY(launch_pdl(attention_decode_kernel<float, false>, grid, dim3(AT_THREADS), 0, stream, p));
  }
  return CUTB_OK;
}
}  // namespace

int attention_decode_launch(int kv_dtype, const float *q, const void *kC, const void *vC, const uint32_t *params, float *out,
                            uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint64_t ld, uint32_t max_seq, float scale,
                            void *workspace, int *status, cudaStream_t stream) {
  if (int rc = check_ld(ld, "attention_decode_launch")) return rc;
  return attention_launch_any(kv_dtype, q, nullptr, nullptr, nullptr, nullptr, const_cast<void *>(kC), const_cast<void *>(vC), params,
                              out, nHeads, nKvHeads, headDim, ld, max_seq, scale, workspace, status, stream);
}

int rope_attention_decode_launch(int kv_dtype, const float *q, const float *k, const float *v, const uint32_t *params,
                                 const float *cosT, const float *sinT, void *kC, void *vC, float *out, uint32_t nHeads,
                                 uint32_t nKvHeads, uint32_t headDim, uint64_t ld, uint32_t max_seq, float scale, void *workspace,
                                 int *status, cudaStream_t stream) {
  if (int rc = check_ld(ld, "rope_attention_decode_launch")) return rc;
  return attention_launch_any(kv_dtype, q, k, v, cosT, sinT, kC, vC, params, out, nHeads, nKvHeads, headDim, ld, max_seq, scale,
                              workspace, status, stream);
}

int batched_kv_write_launch(int kv_dtype, const float *k_in, const float *v_in, uint32_t k_stride, uint32_t v_stride,
                            const uint32_t *positions, const float *cosT, const float *sinT, void *kC, void *vC, uint32_t n_tokens,
                            uint32_t kvDim, uint32_t headDim, uint64_t ld, uint32_t max_seq, int *status, cudaStream_t stream) {
  if (int rc = check_ld(ld, "batched_kv_write_launch")) return rc;
  if (n_tokens == 0) return CUTB_OK;
  if (kv_dtype == CUTB_F16)
    CUTB_CUDA_TRY(launch_pdl(batched_kv_write_kernel<__half>, dim3(n_tokens), dim3(256), 0, stream, k_in, v_in, k_stride, v_stride, positions,
                             cosT, sinT, (__half *)kC, (__half *)vC, kvDim, headDim, (uint32_t)ld, max_seq, status));
  else
    CUTB_CUDA_TRY(launch_pdl(batched_kv_write_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, k_in, v_in, k_stride, v_stride, positions,
                             cosT, sinT, (float *)kC, (float *)vC, kvDim, headDim, (uint32_t)ld, max_seq, status));
  return CUTB_OK;
}

int batched_attention_launch(int kv_dtype, const float *q_in, uint32_t q_stride, const void *kC, const void *vC,
                             const uint32_t *positions, const float *cosT, const float *sinT, float *out, uint32_t out_stride,
                             uint32_t n_tokens, uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint64_t ld, uint32_t max_seq,
                             float scale, int *status, cudaStream_t stream) {
  if (int rc = check_ld(ld, "batched_attention_launch")) return rc;
  if (n_tokens == 0) return CUTB_OK;
  if (batched_attention_tc_applies(kv_dtype, q_in, q_stride, kC, vC, out, out_stride, n_tokens, nHeads, nKvHeads, headDim, ld))
    return batched_attention_tc_launch(q_in, q_stride, kC, vC, positions, cosT, sinT, out, out_stride, n_tokens, nHeads, nKvHeads,
                                       headDim, ld, max_seq, scale, status, stream);
  AttnParams p{};
  p.q = q_in, p.kC = kC, p.vC = vC, p.out = out, p.status = status, p.positions = positions, p.cosT = cosT, p.sinT = sinT;
  p.q_stride = q_stride, p.out_stride = out_stride;
  p.nHeads = nHeads, p.nKvHeads = nKvHeads, p.headDim = headDim, p.ld = (uint32_t)ld, p.nRep = nHeads / nKvHeads;
  p.max_seq = max_seq, p.scale = scale, p.splits = 1;
  p.n_tokens = n_tokens;
  p.tq = (uint32_t)AT_MAX_REP / p.nRep;  // as many tokens per block as the kernel has query-head slots
  if (p.tq < 1) p.tq = 1;
  const uint32_t esz = kv_dtype == CUTB_F16 ? 2 : 4;
  const bool vec = headDim % 32 == 0 && (ld * esz) % 16 == 0 && reinterpret_cast<uintptr_t>(kC) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(vC) % 16 == 0;
  const dim3 grid(nKvHeads, 1, (n_tokens + p.tq - 1) / p.tq);
  if (kv_dtype == CUTB_F16) {
    if (vec) CUTB_CUDA_TRY(launch_pdl(attention_decode_kernel<__half, true>, grid, dim3(AT_THREADS), 0, stream, p));
    else CUTB_CUDA_TRY(launch_pdl(attention_decode_kernel<__half, false>, grid, dim3(AT_THREADS), 0, stream, p));
  } else {
    if (vec) CUTB_CUDA_TRY(launch_pdl(attention_decode_kernel<float, true>, grid, dim3(AT_THREADS), 0, stream, p));
    else CUTB_CUDA_TRY(launch_pdl(attention_decode_kernel<float, false>, grid, dim3(AT_THREADS), 0, stream, p));
  }
  return CUTB_OK;
}

}  // namespace cutb
