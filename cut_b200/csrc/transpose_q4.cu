// Load-time Q4_0 repack: GGML nibble order [N, K/2] -> [K, N/2], low nibble = even n.
//
// Replaces TransposeQ4Nibble.cu (operators/impl/q4transpose/TransposeQ4Nibble.cu:16-61;
// strides from TransposeQ4NibbleOp.cpp:22-23).  In the source, byte j of block b
// of row n holds element 32b + j (low nibble) and 32b + j + 16 (high nibble)
// (interface/loader/gguf/gguf_reader.cpp:559-569).  One thread assembles one
// 32-bit output word = 8 consecutive n at one k; a CTA covers 16 consecutive k
// so that every source byte column of a block is consumed by the same CTA, and
// consecutive lanes write consecutive words.
#include "common.cuh"
#include "kernels.h"

namespace cutb {
namespace {

__global__ void __launch_bounds__(512) transpose_q4_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, uint32_t N,
                                                           uint32_t K, uint32_t stride_in, uint32_t stride_out) {
  const uint32_t halfN = N / 2, words = (halfN + 3) / 4;
  const uint32_t wn = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t k = blockIdx.y * blockDim.y + threadIdx.y;
  if (wn >= words || k >= K) return;
  const uint32_t e = k & 31, col = (k >> 5) * 16 + (e & 15), sh = (e >> 4) * 4;
  uint32_t word = 0;
#pragma unroll
  for (uint32_t i = 0; i < 8; ++i) {
    const uint32_t n = wn * 8 + i;
    if (n < N) word |= ((__ldg(in + (uint64_t)n * stride_in + col) >> sh) & 0xFu) << (4 * i);
  }
  uint8_t *dst = out + (uint64_t)k * stride_out + wn * 4;
  if (wn * 4 + 4 <= halfN && (reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
    *reinterpret_cast<uint32_t *>(dst) = word;
  } else {
    for (uint32_t b = 0; b < 4 && wn * 4 + b < halfN; ++b) dst[b] = (uint8_t)(word >> (8 * b));
  }
}

}  // namespace

int transpose_q4_launch(const void *in, void *out, uint32_t N, uint32_t K, uint32_t stride_in, uint32_t stride_out,
                        cudaStream_t stream) {
  const uint32_t words = (N / 2 + 3) / 4;
  if (words == 0 || K == 0) return CUTB_OK;
  dim3 block(32, 16);
  dim3 grid((words + 31) / 32, (K + 15) / 16);
  transpose_q4_kernel<<<grid, block, 0, stream>>>(reinterpret_cast<const uint8_t *>(in), reinterpret_cast<uint8_t *>(out), N, K,
                                                  stride_in, stride_out);
  CUTB_CUDA_TRY(cudaGetLastError());
  return CUTB_OK;
}

}  // namespace cutb
