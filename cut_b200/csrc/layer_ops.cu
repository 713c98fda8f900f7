// The producer and the consumers of the quantized matmul's operands in a decoder layer: the
// first operators past the matmul path.  RMSNorm (operators/impl/rmsnorm/RMSNorm.cu:6-37),
// embedding row gather (operators/impl/memory/Embedding.cu:18-35) and arg-max / arg-min with the
// reference's tie rule (operators/impl/reduce/ReduceArg.cu:27-59).  All three are bandwidth-
// trivial next to the weight stream (a few KB to a few hundred KB per token).
#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

// One CTA per row: 16-byte loads, the sum of squares in fp32 through a warp-shuffle tree and one
// shared-memory step, y = x * rsqrt(mean + eps) * w.  The row stays in registers between the two
// passes when it fits (up to 8 floats per thread x 256 threads x 4 = 8192 columns); longer rows
// are read twice (the second read hits L2).
template <bool HALF>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const void *__restrict__ x_, const void *__restrict__ w_, void *__restrict__ y_,
                                                      uint32_t dim, uint64_t ldx, float eps) {
  __shared__ float warp_part[8];
  __shared__ float total;
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

// Arg-max / arg-min with the reference's order: a value wins if it is strictly better.  Among
// equal values its 256-thread strided scan keeps each thread's first hit, and its shared-memory
// tree (strides 128, 64, ..., 1, the lower position kept on ties) ends up preferring the thread
// whose index read from the least significant bit upwards is smaller: the winner has the smallest
// bit-reversed (i mod 256), then the smallest i.  The key (value, bitrev8(i mod 256), i) is a
// total order, so any reduction shape gives the same winner: one CTA of 1024 threads.
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
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the reference starts every thread at (worst value, index 0) and replaces it only by strictly
  // better values: an input that never beats the start value yields index 0
  ArgKey best{MAX ? -3.402823466e+38f : 3.402823466e+38f, 0xFFFFFFFFu};
  for (uint32_t i = tid; i < n; i += 1024) {
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
    if (lane == 0) out[0] = best.i == 0xFFFFFFFFu ? 0.0f : (float)best.i;
  }
}

}  // namespace

int rmsnorm_launch(int dtype, const void *x, const void *weight, void *y, uint32_t rows, uint32_t dim, uint64_t ldx, float eps,
                   cudaStream_t stream) {
  if (rows == 0 || dim == 0) return CUTB_OK;
  if (dtype == CUTB_F16)
    rmsnorm_kernel<true><<<rows, 256, 0, stream>>>(x, weight, y, dim, ldx, eps);
  else
    rmsnorm_kernel<false><<<rows, 256, 0, stream>>>(x, weight, y, dim, ldx, eps);
  CUTB_CUDA_TRY(cudaGetLastError());
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
  embedding_kernel<<<(unsigned)blocks, 256, 0, stream>>>(indices, reinterpret_cast<const uint4 *>(table), reinterpret_cast<uint4 *>(out),
                                                         n, ld4, vocab, status);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

int argreduce_launch(int is_max, const float *v, float *out, uint32_t n, cudaStream_t stream) {
  if (is_max)
    argreduce_kernel<true><<<1, 1024, 0, stream>>>(v, out, n);
  else
    argreduce_kernel<false><<<1, 1024, 0, stream>>>(v, out, n);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace cutb
