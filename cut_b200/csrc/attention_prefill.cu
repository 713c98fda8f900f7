// Prefill attention on the tensor cores: a tile of 64 prompt tokens of one query head against the fp16 KV cache.
//
// Same contract as the batched mode of attention_decode_kernel (token i attends cache rows [0, positions[i]] with its
// query rotated here; BatchedAttentionReadCacheOpNode, operators/impl/attention/BatchedAttentionReadCache.cu), which
// serves a few tokens per block with SIMT dot products and took two fifths of a 512-token prefill.  Here a block of
// four warps owns 64 consecutive tokens of one query head: the rotated queries are rounded to fp16 once, K / V tiles of
// 64 cache rows stream through a two-deep cp.async ring, scores and weighted values are m16n8k16 warp MMAs with fp32
// accumulators (a warp owns 16 tokens; the score accumulators are re-packed in registers as the A operand of the
// value product), and the softmax runs online with a running maximum and sum per token, so the only limit on the
// range is the cache itself.  Arithmetic: q and the probabilities are rounded to fp16 (the cache already is), all
// sums are fp32 -- against the SIMT path the output differs by about 1e-3 of its magnitude.
//
// Used for an fp16 cache with head_dim 64 or 128, 16-byte aligned rows and at least 16 tokens; everything else stays
// on the SIMT kernel.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

constexpr int FA_BM = 64;       // tokens per block
constexpr int FA_BN = 64;       // cache rows per tile
constexpr int FA_THREADS = 128;
constexpr int FA_PAD = 8;       // halves of padding per shared row: 16-byte row starts fall on distinct bank groups

struct FaParams {
  const float *q;
  const __half *kC, *vC;
  const uint32_t *positions;
  const float *cosT, *sinT;
  float *out;
  int *status;
  uint32_t q_stride, out_stride, n_tokens, nHeads, nRep, ld, max_seq;
  float scale_log2;  // scale * log2(e): probabilities are 2^(s - m)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D (16x8, fp32) += A (16x16, fp16, row) * B (16x8, fp16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS) batched_attention_tc_kernel(const FaParams p) {
  constexpr int LDS = HD + FA_PAD;             // halves per shared row
  constexpr int KS = HD / 16;                  // k steps of the score product
  constexpr uint32_t TILE = FA_BN * LDS * 2;   // bytes of one K or V tile
  extern __shared__ __align__(16) uint8_t fa_smem[];
  __half *Qs = reinterpret_cast<__half *>(fa_smem);                   // [FA_BM][LDS]
  const uint32_t qs_u = smem_u32(fa_smem), k_u = qs_u + FA_BM * LDS * 2, v_u = k_u + 2 * TILE;  // K[2], V[2]
  __shared__ uint32_t pos_s[FA_BM];   // cache row of each token; 0xFFFFFFFF: no such token
  __shared__ uint32_t kv_len_s;

  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t tok0 = blockIdx.x * FA_BM, h = blockIdx.y, kvh = h / p.nRep;
  pdl_enter();  // q, the caches and the positions may come from the kernels before

  if (tid == 0) kv_len_s = 0;
  __syncthreads();
  if (tid < FA_BM) {
    uint32_t pos = 0xFFFFFFFFu;
    if (tok0 + tid < p.n_tokens) {
      pos = __ldg(p.positions + tok0 + tid);
      if (pos >= p.max_seq) {  // never read outside the cache
        if (p.status && h == 0) atomicExch(p.status, (int)CUTB_ERR_INVALID);
        pos = p.max_seq - 1;
      }
      atomicMax(&kv_len_s, pos + 1);
    }
    pos_s[tid] = pos;
  }
  __syncthreads();
  const uint32_t kv_len = kv_len_s, ntiles = (kv_len + FA_BN - 1) / FA_BN;

  // one tile = FA_BN cache rows x HD halves of this KV head; rows past the attended range are zero (a masked score is
  // overwritten, but a probability of zero times a stray NaN in V would not be zero)
  const __half *kbase = p.kC + (size_t)kvh * HD, *vbase = p.vC + (size_t)kvh * HD;
  auto load_tile = [&](uint32_t t, uint32_t buf) {
    constexpr int CH = HD / 8;  // 16-byte chunks per row
    for (uint32_t i = tid; i < FA_BN * CH; i += FA_THREADS) {
      const uint32_t r = i / CH, c = i % CH, row = t * FA_BN + r;
      const uint32_t off = (r * LDS + c * 8) * 2;
      if (row < kv_len) {
        cp_async16(k_u + buf * TILE + off, kbase + (size_t)row * p.ld + c * 8);
        cp_async16(v_u + buf * TILE + off, vbase + (size_t)row * p.ld + c * 8);
      } else {
        *reinterpret_cast<uint4 *>(fa_smem + (k_u - qs_u) + buf * TILE + off) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4 *>(fa_smem + (v_u - qs_u) + buf * TILE + off) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };
  if (ntiles) load_tile(0, 0);

  // queries: rotate at the token's own position (half-split; products and sums rounded separately, as
  // BatchedAttentionReadCache does), round to fp16
  {
    constexpr uint32_t half = HD / 2;
    for (uint32_t i = tid; i < FA_BM * HD; i += FA_THREADS) {
      const uint32_t r = i / HD, e = i % HD;
      float val = 0.f;
      const uint32_t pos = pos_s[r];
      if (pos != 0xFFFFFFFFu) {
        const float *x = p.q + (size_t)(tok0 + r) * p.q_stride + (size_t)h * HD + e;
        const float *cs = p.cosT + (size_t)pos * half, *sn = p.sinT + (size_t)pos * half;
        val = e < half ? __fsub_rn(__fmul_rn(__ldg(x), __ldg(cs + e)), __fmul_rn(__ldg(x + half), __ldg(sn + e)))
                       : __fadd_rn(__fmul_rn(__ldg(x - half), __ldg(sn + e - half)), __fmul_rn(__ldg(x), __ldg(cs + e - half)));
      }
      Qs[r * LDS + e] = __float2half_rn(val);
    }
  }
  __syncthreads();

  // this warp's 16 tokens as A fragments, kept for every tile
  const uint32_t g = lane >> 2, tg = lane & 3, mat = lane >> 3, mr = lane & 7;
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    // matrices: (rows 0-7, k 0-7) (rows 8-15, k 0-7) (rows 0-7, k 8-15) (rows 8-15, k 8-15)
    const uint32_t row = warp * 16 + (mat & 1) * 8 + mr, col = ks * 16 + (mat >> 1) * 8;
    ldsm_x4(qs_u + (row * LDS + col) * 2, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
  }
  const uint32_t row_lo = warp * 16 + g, row_hi = row_lo + 8;
  const uint32_t pos_lo = pos_s[row_lo], pos_hi = pos_s[row_hi];

  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;  // running maximum (in log2 units) and sum per token

  for (uint32_t t = 0; t < ntiles; ++t) {
    const uint32_t buf = t & 1;
    if (t + 1 < ntiles) {
      load_tile(t + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kt_u = k_u + buf * TILE, vt_u = v_u + buf * TILE;

    // scores: 16 tokens x 64 rows
    float s[FA_BN / 8][4];
#pragma unroll
    for (int j = 0; j < FA_BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int j2 = 0; j2 < FA_BN / 16; ++j2) {
        // matrices: (rows 16 j2 + 0-7, k 0-7) (same rows, k 8-15) (rows 16 j2 + 8-15, k 0-7) (those rows, k 8-15)
        const uint32_t row = j2 * 16 + (mat >> 1) * 8 + mr, col = ks * 16 + (mat & 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kt_u + (row * LDS + col) * 2, b0, b1, b2, b3);
        mma_16816(s[2 * j2], qa[ks], b0, b1);
        mma_16816(s[2 * j2 + 1], qa[ks], b2, b3);
      }
    }
    // scale, mask (a row beyond the token's own position; a token that does not exist), running maximum
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < FA_BN / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t key = t * FA_BN + j * 8 + 2 * tg + (e & 1);
        const uint32_t pos = e < 2 ? pos_lo : pos_hi;
        const bool ok = pos != 0xFFFFFFFFu && key <= pos;
        const float v = ok ? s[j][e] * p.scale_log2 : -INFINITY;
        s[j][e] = v;
        if (e < 2) mx_lo = fmaxf(mx_lo, v);
        else mx_hi = fmaxf(mx_hi, v);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    // nothing attended yet (a padding token): keep exponents finite
    const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    const float al_lo = exp2f(m_lo - ms_lo), al_hi = exp2f(m_hi - ms_hi);  // 0 while the old maximum is -inf
    m_lo = mn_lo, m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int j = 0; j < FA_BN / 8; ++j) {
      s[j][0] = exp2f(s[j][0] - ms_lo), s[j][1] = exp2f(s[j][1] - ms_lo);
      s[j][2] = exp2f(s[j][2] - ms_hi), s[j][3] = exp2f(s[j][3] - ms_hi);
      sum_lo += s[j][0] + s[j][1];
      sum_hi += s[j][2] + s[j][3];
    }
    l_lo = l_lo * al_lo + sum_lo, l_hi = l_hi * al_hi + sum_hi;  // this thread's share of the row; met at the end
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) o[j][0] *= al_lo, o[j][1] *= al_lo, o[j][2] *= al_hi, o[j][3] *= al_hi;

    // weighted values: the probabilities of 16 rows are the A operand as they lie in the accumulators
#pragma unroll
    for (int kk = 0; kk < FA_BN / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_h2(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_h2(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jd2 = 0; jd2 < HD / 16; ++jd2) {
        // transposed 8x8 loads: (rows 16 kk + 0-7, dims 0-7) (rows + 8-15, dims 0-7) (rows 0-7, dims 8-15) (rows 8-15, dims 8-15)
        const uint32_t row = kk * 16 + (mat & 1) * 8 + mr, col = jd2 * 16 + (mat >> 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(vt_u + (row * LDS + col) * 2, b0, b1, b2, b3);
        mma_16816(o[2 * jd2], pa, b0, b1);
        mma_16816(o[2 * jd2 + 1], pa, b2, b3);
      }
    }
    __syncthreads();  // the tile is free for the copy issued two iterations from now
  }

  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = l_lo > 0.f ? 1.0f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.0f / l_hi : 0.f;
  if (pos_lo != 0xFFFFFFFFu) {
    float *dst = p.out + (size_t)(tok0 + row_lo) * p.out_stride + (size_t)h * HD + 2 * tg;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) *reinterpret_cast<float2 *>(dst + 8 * j) = make_float2(o[j][0] * inv_lo, o[j][1] * inv_lo);
  }
  if (pos_hi != 0xFFFFFFFFu) {
    float *dst = p.out + (size_t)(tok0 + row_hi) * p.out_stride + (size_t)h * HD + 2 * tg;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) *reinterpret_cast<float2 *>(dst + 8 * j) = make_float2(o[j][2] * inv_hi, o[j][3] * inv_hi);
  }
}

template <int HD> int fa_launch(const FaParams &p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)(FA_BM + 4 * FA_BN) * (HD + FA_PAD) * 2;
  static bool configured[64] = {};  // per device: the attribute is set once on each
  int dev = 0;
  CUTB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    CUTB_CUDA_TRY(cudaFuncSetAttribute(batched_attention_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const dim3 grid((p.n_tokens + FA_BM - 1) / FA_BM, p.nHeads);
  CUTB_CUDA_TRY(launch_pdl(batched_attention_tc_kernel<HD>, grid, dim3(FA_THREADS), smem, stream, p));
  return CUTB_OK;
}

}  // namespace

bool batched_attention_tc_applies(int kv_dtype, const float *q_in, uint32_t q_stride, const void *kC, const void *vC, const float *out,
                                  uint32_t out_stride, uint32_t n_tokens, uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim,
                                  uint64_t ld) {
  (void)q_in;
  (void)q_stride;
  if (kv_dtype != CUTB_F16 || (headDim != 64 && headDim != 128) || n_tokens < 16) return false;
  if (nKvHeads == 0 || nHeads % nKvHeads != 0) return false;
  // 16-byte cache rows for cp.async, 8-byte output pairs
  if ((ld * 2) % 16 != 0 || reinterpret_cast<uintptr_t>(kC) % 16 != 0 || reinterpret_cast<uintptr_t>(vC) % 16 != 0) return false;
  if (reinterpret_cast<uintptr_t>(out) % 8 != 0 || out_stride % 2 != 0) return false;
  return true;
}

int batched_attention_tc_launch(const float *q_in, uint32_t q_stride, const void *kC, const void *vC, const uint32_t *positions,
                                const float *cosT, const float *sinT, float *out, uint32_t out_stride, uint32_t n_tokens,
                                uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint64_t ld, uint32_t max_seq, float scale,
                                int *status, cudaStream_t stream) {
  FaParams p{};
  p.q = q_in, p.kC = reinterpret_cast<const __half *>(kC), p.vC = reinterpret_cast<const __half *>(vC);
  p.positions = positions, p.cosT = cosT, p.sinT = sinT, p.out = out, p.status = status;
  p.q_stride = q_stride, p.out_stride = out_stride, p.n_tokens = n_tokens, p.nHeads = nHeads, p.nRep = nHeads / nKvHeads;
  p.ld = (uint32_t)ld, p.max_seq = max_seq;
  p.scale_log2 = scale * 1.4426950408889634f;
  return headDim == 128 ? fa_launch<128>(p, stream) : fa_launch<64>(p, stream);
}

}  // namespace cutb
