// The producer and the consumers of the quantized matmul's operands in a decoder layer: the
// first operators past the matmul path.  RMSNorm (operators/impl/rmsnorm/RMSNorm.cu:6-37),
// embedding row gather (operators/impl/memory/Embedding.cu:18-35) and arg-max / arg-min with the
// reference's tie rule (operators/impl/reduce/ReduceArg.cu:27-59).  All three are bandwidth-
// trivial next to the weight stream (a few KB to a few hundred KB per token).
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace cutb {
namespace {

// fp32 rows of up to 8192 columns whose length and stride are multiples of 4: one CTA of up to
// 1024 threads per row, every thread loads its (at most two) 16-byte pieces of the row and of the
// weight at once, so the whole operator is one memory round trip, a shuffle tree and two barriers;
// the row never leaves registers.
__global__ void __launch_bounds__(1024) rmsnorm_row_kernel(const float4 *__restrict__ x, const float4 *__restrict__ w,
                                                           float4 *__restrict__ y, uint32_t dim4, uint64_t ldx4, float inv_dim,
                                                           float eps) {
  __shared__ float warp_part[32];
  pdl_enter();
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const uint64_t row = blockIdx.x;
  const uint32_t i0 = tid, i1 = tid + blockDim.x;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 a0 = i0 < dim4 ? __ldg(x + row * ldx4 + i0) : zero, a1 = i1 < dim4 ? __ldg(x + row * ldx4 + i1) : zero;
  const float4 w0 = i0 < dim4 ? __ldg(w + i0) : zero, w1 = i1 < dim4 ? __ldg(w + i1) : zero;
  float ss = fmaf(a0.x, a0.x, fmaf(a0.y, a0.y, fmaf(a0.z, a0.z, a0.w * a0.w)));
  ss += fmaf(a1.x, a1.x, fmaf(a1.y, a1.y, fmaf(a1.z, a1.z, a1.w * a1.w)));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if (lane == 0) warp_part[warp] = ss;
  __syncthreads();
  float t = lane < nwarps ? warp_part[lane] : 0.f;  // every warp adds the partials in the same order
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
  const float scale = rsqrtf(t * inv_dim + eps);
  if (i0 < dim4) y[row * ldx4 + i0] = make_float4(a0.x * scale * w0.x, a0.y * scale * w0.y, a0.z * scale * w0.z, a0.w * scale * w0.w);
  if (i1 < dim4) y[row * ldx4 + i1] = make_float4(a1.x * scale * w1.x, a1.y * scale * w1.y, a1.z * scale * w1.z, a1.w * scale * w1.w);
}

// Any other row: one CTA of 256 threads per row, the sum of squares in fp32 through a
// warp-shuffle tree and one shared-memory step, y = x * rsqrt(mean + eps) * w; the row is read
// twice (the second read hits L2).
template <bool HALF>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const void *__restrict__ x_, const void *__restrict__ w_, void *__restrict__ y_,
                                                      uint32_t dim, uint64_t ldx, float eps) {
  __shared__ float warp_part[8];
  __shared__ float total;
  pdl_enter();
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint64_t row = blockIdx.x;
  auto ldx_at = [&](uint32_t i) -> float {
    if constexpr (HALF) return __half2float(__ldg(reinterpret_cast<const __half *>(x_) + row * ldx + i));
    return __ldg(reinterpret_cast<const float *>(x_) + row * ldx + i);
  };
  auto ldw_at = [&](uint32_t i) -> float {
    if constexpr (HALF) return __half2float(__ldg(reinterpret_cast<const __half *>(w_) + i));
    return __ldg(reinterpret_cast<const float *>(w_) + i);
  };
  float ss = 0.f;
  for (uint32_t i = tid; i < dim; i += 256) {
    const float v = ldx_at(i);
    ss = fmaf(v, v, ss);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_down_sync(0xffffffffu, ss, off);
  if (lane == 0) warp_part[warp] = ss;
  __syncthreads();
  if (tid == 0) {
    float t = warp_part[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += warp_part[w];
    total = t;
  }
  __syncthreads();
  const float scale = rsqrtf(total / (float)dim + eps);
  for (uint32_t i = tid; i < dim; i += 256) {
    const float out = ldx_at(i) * scale * ldw_at(i);
    if constexpr (HALF)
      reinterpret_cast<__half *>(y_)[row * ldx + i] = __float2half_rn(out);
    else
      reinterpret_cast<float *>(y_)[row * ldx + i] = out;
  }
}

// out[i, :] = table[indices[i], :] in 16-byte pieces; ld4 = row length in 16-byte pieces.
__global__ void __launch_bounds__(256) embedding_kernel(const uint32_t *__restrict__ indices, const uint4 *__restrict__ table,
                                                        uint4 *__restrict__ out, uint64_t n, uint32_t ld4, uint32_t vocab,
                                                        int *status) {
  pdl_enter();
  const uint64_t total = n * ld4;
  for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t i = g / ld4;
    const uint32_t c = (uint32_t)(g % ld4);
    const uint32_t row = __ldg(indices + i);
    if (row >= vocab) {  // never read outside the table: record it and write zeros
      if (status) atomicExch(status, (int)CUTB_ERR_INVALID);
      out[g] = make_uint4(0, 0, 0, 0);
      continue;
    }
    out[g] = __ldg(table + (uint64_t)row * ld4 + c);
  }
}

// Column gather from a [dim, vocab] matrix: out[i, d] = M[d, indices[i]] -- the embedding read out of a
// tied LM head that is stored in the matmul's [K, N] orientation (operators/impl/memory/EmbeddingCol.cu:16-44).
// format 0: fp16 matrix; format 1: int8 values with one fp16 scale per 32 rows and column
// (scales [dim / 32, vocab]).  An index >= vocab writes zeros and reports through *status.
__global__ void __launch_bounds__(256) embedding_col_kernel(const uint32_t *__restrict__ indices, const void *__restrict__ matrix,
                                                            const __half *__restrict__ scales, float *__restrict__ out, uint32_t n,
                                                            uint32_t dim, uint32_t vocab, uint32_t vocab_stride, uint32_t scale_stride,
                                                            uint32_t out_stride, int format, int *status) {
  pdl_enter();
  const uint64_t total = (uint64_t)n * dim;
  for (uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total; gid += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t i = (uint32_t)(gid / dim), d = (uint32_t)(gid % dim);
    const uint32_t tkn = __ldg(indices + i);
    float v = 0.f;
    if (tkn >= vocab) {
      if (status) atomicExch(status, (int)CUTB_ERR_INVALID);
    } else if (format == 0) {
      v = __half2float(__ldg(reinterpret_cast<const __half *>(matrix) + (uint64_t)d * vocab_stride + tkn));
    } else {
      const int b = (int)__ldg(reinterpret_cast<const int8_t *>(matrix) + (uint64_t)d * vocab_stride + tkn);
      v = (float)b * __half2float(__ldg(scales + (uint64_t)(d >> 5) * scale_stride + tkn));
    }
    out[(uint64_t)i * out_stride + d] = v;
  }
}

// Arg-max / arg-min with the reference's order: a value wins if it is strictly better.  Among
// equal values its 256-thread strided scan keeps each thread's first hit, and its shared-memory
// tree (strides 128, 64, ..., 1, the lower position kept on ties) ends up preferring the thread
// whose index read from the least significant bit upwards is smaller: the winner has the smallest
// bit-reversed (i mod 256), then the smallest i.  The key (value, bitrev8(i mod 256), i) is a
// total order, so any reduction shape gives the same winner: one CTA of 1024 threads, or for long inputs
// (a vocabulary of logits) a cluster of eight whose block winners meet through distributed shared memory.
struct ArgKey {
  float v;
  uint32_t i;
};
template <bool MAX> __device__ __forceinline__ bool arg_better(const ArgKey &a, const ArgKey &b) {
  if (a.v != b.v) return MAX ? a.v > b.v : a.v < b.v;
  const uint32_t ta = __brev(a.i & 255u), tb = __brev(b.i & 255u);  // bit-reversed thread index of the reference's scan
  if (ta != tb) return ta < tb;
  return a.i < b.i;
}
template <bool MAX>
__global__ void __launch_bounds__(1024) argreduce_kernel(const float *__restrict__ v, float *__restrict__ out, uint32_t n) {
  __shared__ ArgKey part[32];
  __shared__ ArgKey block_best;
  pdl_enter();
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the reference starts every thread at (worst value, index 0) and replaces it only by strictly
  // better values: an input that never beats the start value yields index 0
  ArgKey best{MAX ? -3.402823466e+38f : 3.402823466e+38f, 0xFFFFFFFFu};
  const uint32_t step = gridDim.x * 1024;
#pragma unroll 4
  for (uint32_t i = blockIdx.x * 1024 + tid; i < n; i += step) {
    const ArgKey c{__ldg(v + i), i};
    const bool strictly = MAX ? c.v > best.v : c.v < best.v;
    if (strictly || (c.v == best.v && best.i != 0xFFFFFFFFu && arg_better<MAX>(c, best))) best = c;
  }
  auto merge = [&](ArgKey o) {
    if (o.i == 0xFFFFFFFFu) return;
    if (best.i == 0xFFFFFFFFu || arg_better<MAX>(o, best)) best = o;
  };
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    ArgKey o;
    o.v = __shfl_down_sync(0xffffffffu, best.v, off);
    o.i = __shfl_down_sync(0xffffffffu, best.i, off);
    merge(o);
  }
  if (lane == 0) part[warp] = best;
  __syncthreads();
  if (warp == 0) {
    best = part[lane];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      ArgKey o;
      o.v = __shfl_down_sync(0xffffffffu, best.v, off);
      o.i = __shfl_down_sync(0xffffffffu, best.i, off);
      merge(o);
    }
    if (lane == 0) {
      if (gridDim.x == 1) out[0] = best.i == 0xFFFFFFFFu ? 0.0f : (float)best.i;
      else block_best = best;
    }
  }
  if (gridDim.x > 1) {  // launched as one cluster: block 0 collects the block winners
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (blockIdx.x == 0 && tid == 0) {
      best = block_best;
      for (uint32_t r = 1; r < gridDim.x; ++r) merge(*cluster.map_shared_rank(&block_best, r));
      out[0] = best.i == 0xFFFFFFFFu ? 0.0f : (float)best.i;
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
  }
}

// out[r, i] = unary(in[r, 2i]) * in[r, 2i + 1]: the gated feed-forward's activation over a prefill GEMM whose
// weight rows are stored in (gate, up) pairs (the decode mat-vec does this in its epilogue).
__global__ void __launch_bounds__(256) glu_pairs_kernel(const float2 *__restrict__ in, float *__restrict__ out, uint32_t rows,
                                                        uint32_t cols_out, uint64_t ldi2, uint64_t ldo, int op) {
  pdl_enter();
  const uint64_t total = (uint64_t)rows * cols_out;
  for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t r = g / cols_out, c = g % cols_out;
    const float2 gu = __ldg(in + r * ldi2 + c);
    out[r * ldo + c] = apply_epilogue(gu.x, CUTB_FUSION_UNARY, op, 0.f) * gu.y;
  }
}

}  // namespace

int glu_pairs_launch(const float *in, float *out, uint32_t rows, uint32_t cols_out, uint64_t ldi, uint64_t ldo, int unary_op,
                     cudaStream_t stream) {
  const uint64_t total = (uint64_t)rows * cols_out;
  if (total == 0) return CUTB_OK;
  uint64_t blocks = (total + 255) / 256;
  DeviceInfo di;
  const uint64_t sms = (get_device_info(&di) == CUTB_OK && di.sm_count > 0) ? (uint64_t)di.sm_count : 148u;
  if (blocks > sms * 16) blocks = sms * 16;
  CUTB_CUDA_TRY(launch_pdl(glu_pairs_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, reinterpret_cast<const float2 *>(in), out, rows,
                           cols_out, ldi / 2, ldo, unary_op));
  return CUTB_OK;
}

int rmsnorm_launch(int dtype, const void *x, const void *weight, void *y, uint32_t rows, uint32_t dim, uint64_t ldx, float eps,
                   cudaStream_t stream) {
  if (rows == 0 || dim == 0) return CUTB_OK;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (dtype == CUTB_F32 && aligned && dim % 4 == 0 && ldx % 4 == 0 && dim <= 8192) {
    const uint32_t dim4 = dim / 4;
    uint32_t threads = ((dim4 + 1) / 2 + 31) / 32 * 32;  // two pieces per thread, whole warps
    if (threads < 128) threads = (dim4 + 31) / 32 * 32 < 128 ? (dim4 + 31) / 32 * 32 : 128;
    CUTB_CUDA_TRY(launch_pdl(rmsnorm_row_kernel, dim3(rows), dim3(threads), 0, stream, reinterpret_cast<const float4 *>(x),
                             reinterpret_cast<const float4 *>(weight), reinterpret_cast<float4 *>(y), dim4, ldx / 4, 1.0f / (float)dim,
                             eps));
  } else if (dtype == CUTB_F16)
    CUTB_CUDA_TRY(launch_pdl(rmsnorm_kernel<true>, dim3(rows), dim3(256), 0, stream, x, weight, y, dim, ldx, eps));
  else
    CUTB_CUDA_TRY(launch_pdl(rmsnorm_kernel<false>, dim3(rows), dim3(256), 0, stream, x, weight, y, dim, ldx, eps));
  return CUTB_OK;
}

int embedding_launch(const uint32_t *indices, const float *table, float *out, uint64_t n, uint32_t dim, uint32_t vocab, int *status,
                     cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  const uint32_t ld4 = (dim + 3) / 4;
  const uint64_t total = n * ld4;
  if (total == 0) return CUTB_OK;
  uint64_t blocks = (total + 255) / 256;
  if (blocks > (uint64_t)di.sm_count * 16) blocks = (uint64_t)di.sm_count * 16;
  CUTB_CUDA_TRY(launch_pdl(embedding_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, indices, reinterpret_cast<const uint4 *>(table),
                           reinterpret_cast<uint4 *>(out), n, ld4, vocab, status));
  return CUTB_OK;
}

int embedding_col_launch(int format, const uint32_t *indices, const void *matrix, const void *scales, float *out, uint32_t n,
                         uint32_t dim, uint32_t vocab, uint32_t vocab_stride, uint32_t scale_stride, uint32_t out_stride, int *status,
                         cudaStream_t stream) {
  DeviceInfo di;
  if (int rc = get_device_info(&di)) return rc;
  const uint64_t total = (uint64_t)n * dim;
  if (total == 0) return CUTB_OK;
  uint64_t blocks = (total + 255) / 256;
  if (blocks > (uint64_t)di.sm_count * 16) blocks = (uint64_t)di.sm_count * 16;
  CUTB_CUDA_TRY(launch_pdl(embedding_col_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, indices, matrix,
                           reinterpret_cast<const __half *>(scales), out, n, dim, vocab, vocab_stride, scale_stride, out_stride, format,
                           status));
  return CUTB_OK;
}

int argreduce_launch(int is_max, const float *v, float *out, uint32_t n, cudaStream_t stream) {
  if (n >= 8192) {  // eight blocks as one cluster
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(8);
    cfg.blockDim = dim3(1024);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 8;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (is_max)
      CUTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, argreduce_kernel<true>, v, out, n));
    else
      CUTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, argreduce_kernel<false>, v, out, n));
    return CUTB_OK;
  }
  if (is_max)
    CUTB_CUDA_TRY(launch_pdl(argreduce_kernel<true>, dim3(1), dim3(1024), 0, stream, v, out, n));
  else
    CUTB_CUDA_TRY(launch_pdl(argreduce_kernel<false>, dim3(1), dim3(1024), 0, stream, v, out, n));
  return CUTB_OK;
}

// ---- batched device copies ----------------------------------------------------------------------
// One launch moves n byte ranges device -> device: blockIdx.y = range, blockIdx.x strides over its 16-byte
// vectors.  A backend uses it to scatter one coalesced host upload into the tensors it belongs to, and to gather
// a step's results into one block for a single download.  The table may live in host-mapped pinned memory (it
// is read once per block).
__global__ void __launch_bounds__(256) copy_batch_kernel(const cutb_copy_range *__restrict__ table) {
  const cutb_copy_range r = table[blockIdx.y];
  const uint64_t vecs = r.bytes / 16;
  const uint4 *src = reinterpret_cast<const uint4 *>(r.src);
  uint4 *dst = reinterpret_cast<uint4 *>(r.dst);
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (uint64_t)gridDim.x * blockDim.x) dst[i] = src[i];
  if (blockIdx.x == 0) {  // tail bytes (ranges need not be multiples of 16)
    const uint8_t *s8 = reinterpret_cast<const uint8_t *>(r.src);
    uint8_t *d8 = reinterpret_cast<uint8_t *>(r.dst);
    for (uint64_t i = vecs * 16 + threadIdx.x; i < r.bytes; i += blockDim.x) d8[i] = s8[i];
  }
}

int copy_batch_launch(const cutb_copy_range *table, uint32_t n, uint32_t blocks_per_range, cudaStream_t stream) {
  copy_batch_kernel<<<dim3(blocks_per_range, n), 256, 0, stream>>>(table);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace cutb
