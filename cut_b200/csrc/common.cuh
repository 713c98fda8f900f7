// Shared device/host helpers of the sm_100a quantized-matmul kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cutb.h"

namespace cutb {

// ---------------------------------------------------------------------------
// Host-side error plumbing (the C ABI never throws).
// ---------------------------------------------------------------------------
void set_last_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define CUTB_CUDA_TRY(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::cutb::cuda_fail(_e, #expr); \
  } while (0)

// Block geometry of the three GGUF formats the path covers
// (interface/loader/gguf/gguf_types.hpp:109-150).
__host__ __device__ constexpr uint32_t block_elems(int fmt) {
  return (fmt == CUTB_Q4_K || fmt == CUTB_Q5_K || fmt == CUTB_Q6_K) ? 256u : (fmt == CUTB_BF16 ? 1u : 32u);
}
__host__ __device__ constexpr uint32_t block_bytes(int fmt) {
  return fmt == CUTB_Q8_0 ? 34u : fmt == CUTB_Q4_0 ? 18u : fmt == CUTB_Q4_K ? 144u : fmt == CUTB_Q5_K ? 176u : fmt == CUTB_Q6_K ? 210u
         : fmt == CUTB_Q4_1 ? 20u : fmt == CUTB_Q5_0 ? 22u : 2u;
}
// Bytes of 256 consecutive weights of one row: the copy granule of the decode
// kernel (a multiple of 16 bytes in all three formats).
__host__ __device__ constexpr uint32_t granule_bytes(int fmt) { return fmt == CUTB_Q8_0 ? 272u : 144u; }

inline uint64_t row_bytes(int fmt, uint32_t K) {
  return (uint64_t)((K + block_elems(fmt) - 1) / block_elems(fmt)) * block_bytes(fmt);
}

// Cached device properties of the current device.
struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t smem_optin = 0;
  size_t smem_per_sm = 0;
};
int get_device_info(DeviceInfo *out);

// ---------------------------------------------------------------------------
// Device helpers.
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

// fp16 bits -> float, subnormals decoded, exactly as the reference's loader does
// (interface/loader/gguf/gguf_reader.cpp:515-539); the hardware conversion is
// exact for every fp16 value, subnormals included.
__device__ __forceinline__ float h2f_bits(uint32_t bits) {
  return __half2float(__ushort_as_half((unsigned short)bits));
}

// Fused epilogue of the reference's quantized matmul
// (operators/impl/matmul/MatMulQ4Common.cuh:63-114): unary ops on the result,
// or binary ops against the D operand.  One list of op codes and expressions serves
// the one-value form and the N-value form below, so both produce the same bits.
#define CUTB_UNARY_OPS(X)                                                                                          \
  X(100, -x)                                                                                                       \
  X(101, fabsf(x))                                                                                                 \
  X(102, sqrtf(x))                                                                                                 \
  X(103, x * x)                                                                                                    \
  X(104, 1.0f / x)                                                                                                 \
  X(106, expf(x))                                                                                                  \
  X(109, logf(x))                                                                                                  \
  X(121, tanhf(x))                                                                                                 \
  X(122, floorf(x))                                                                                                \
  X(123, ceilf(x))                                                                                                 \
  X(124, roundf(x))                                                                                                \
  X(130, fmaxf(0.0f, x))                                                                                           \
  X(131, 1.0f / (1.0f + expf(-x)))                                                                                 \
  X(132, x * 0.5f * (1.0f + tanhf(sqrtf(2.0f / 3.14159265f) * (x + 0.044715f * x * x * x))))                      \
  X(133, x / (1.0f + expf(-x)))                                                                                    \
  X(134, logf(1.0f + expf(x)))                                                                                     \
  X(137, fminf(fmaxf(x, 0.0f), 6.0f))                                                                              \
  X(141, x * tanhf(logf(1.0f + expf(x))))                                                                          \
  X(142, x * fminf(fmaxf(x / 6.0f + 0.5f, 0.0f), 1.0f))                                                            \
  X(143, fminf(fmaxf(x / 6.0f + 0.5f, 0.0f), 1.0f))                                                                \
  X(148, rsqrtf(x))
#define CUTB_BINARY_OPS(X)                                                                                         \
  X(0, a + b)                                                                                                      \
  X(1, a - b)                                                                                                      \
  X(2, a * b)                                                                                                      \
  X(3, a / b)                                                                                                      \
  X(4, a - b * floorf(a / b))                                                                                      \
  X(5, powf(a, b))                                                                                                 \
  X(6, floorf(a / b))                                                                                              \
  X(13, fminf(a, b))                                                                                               \
  X(14, fmaxf(a, b))

__device__ __forceinline__ float apply_epilogue(float v, int type, int op, float d) {
  if (type == CUTB_FUSION_UNARY) {
    const float x = v;
    switch (op) {
#define CUTB_CASE(code, expr) \
  case code: return (expr);
      CUTB_UNARY_OPS(CUTB_CASE)
#undef CUTB_CASE
      default: return x;
    }
  }
  if (type == CUTB_FUSION_BINARY) {
    const float a = v, b = d;
    switch (op) {
#define CUTB_CASE(code, expr) \
  case code: return (expr);
      CUTB_BINARY_OPS(CUTB_CASE)
#undef CUTB_CASE
      default: return a + b;
    }
  }
  return v;
}

// The same on N values held in registers, with the op selected once outside the loop: an unrolled loop around the
// one-value form repeats the whole switch N times, which is more code than the instruction cache holds (a fused
// SiLU made the 512-token GEMM's epilogue three times slower than the whole unfused kernel).
template <int N> __device__ __forceinline__ void apply_epilogue_n(float (&v)[N], const float (&d)[N], int type, int op) {
  if (type == CUTB_FUSION_UNARY) {
    switch (op) {
#define CUTB_CASE(code, expr)         \
  case code:                          \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { \
      const float x = v[i];           \
      v[i] = (expr);                  \
    }                                 \
    break;
      CUTB_UNARY_OPS(CUTB_CASE)
#undef CUTB_CASE
      default: break;
    }
  } else if (type == CUTB_FUSION_BINARY) {
    switch (op) {
#define CUTB_CASE(code, expr)         \
  case code:                          \
    _Pragma("unroll") for (int i = 0; i < N; ++i) { \
      const float a = v[i], b = d[i]; \
      v[i] = (expr);                  \
    }                                 \
    break;
      CUTB_BINARY_OPS(CUTB_CASE)
#undef CUTB_CASE
      default:
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = v[i] + d[i];
        break;
    }
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier + bulk async copy (TMA engine, untiled form) ------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One try_wait with a suspend-time hint: the hardware parks the thread until the
// phase completes or about `hint_ns` nanoseconds pass, so a waiting warp issues
// almost no instructions (a hot polling loop competes for issue slots with the
// warps that do the work).
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` parked waits of up to ~16 us each (about a
// second by default) and returns false; the caller records CUTB_ERR_TIMEOUT and
// drains instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 16)) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity, 16384u)) return true;
  return false;
}
// Probe once, park only if the phase is still open: a parked wait costs a few hundred
// cycles even when the barrier completed long ago, the probe a few tens.  (Polling in a
// loop instead of parking was slower in the decode kernel: the pollers of both resident
// CTAs take issue slots from the warps that compute.)
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_probe_first(uint32_t bar, uint32_t parity) {
  return mbar_test(bar, parity) || mbar_wait_bounded(bar, parity);
}
// Bounded polling wait without parking: for the single threads on a kernel's critical
// path (an MMA issuer, a copy producer), where the wake-up delay of a parked wait would
// be paid once per pipeline step.  About a second at ~30 cycles per probe.
__device__ __forceinline__ bool mbar_spin_bounded(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 26)) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// global -> this CTA's shared memory, completion counted in bytes on `bar`.
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// llama.cpp:445-482: float -> half with the dropped bits rounded half UP, subnormals encoded,
// overflow to infinity (NaN is not special-cased there and becomes infinity too).
__device__ __forceinline__ uint16_t f32_to_f16_runner(float v) {
  const uint32_t u = __float_as_uint(v);
  const uint32_t sign = (u >> 16) & 0x8000u;
  int32_t e = (int32_t)((u >> 23) & 0xffu) - 127 + 15;
  const uint32_t mantissa = u & 0x7fffffu;
  if (e <= 0) {
    const uint32_t shift = (uint32_t)(14 - e);
    if (shift > 24) return (uint16_t)sign;
    const uint32_t significand = 0x800000u | mantissa;
    uint32_t half = significand >> shift;
    if ((significand >> (shift - 1)) & 1u) ++half;
    return (uint16_t)(sign | half);
  }
  if (e >= 31) return (uint16_t)(sign | 0x7c00u);
  uint32_t m = mantissa >> 13;
  if (mantissa & 0x1000u) {
    ++m;
    if (m == 0x400u) {
      m = 0;
      ++e;
      if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    }
  }
  return (uint16_t)(sign | ((uint32_t)e << 10) | m);
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

#endif  // __CUDACC__

// Programmatic dependent launch for the small kernels of a decode step.  A kernel launched with
// programmatic stream serialization may be scheduled while its predecessor in the stream still
// runs (when that predecessor releases it early, as the decode mat-vec does); pdl_enter() waits
// until the predecessor grid has completed and its writes are visible.  Nothing is read or
// written before it, so stream order is kept; what overlaps is launch latency and block
// scheduling.  The small kernels do not release their own successor early: measured on a whole
// decoder step, mat-vecs that start under a small kernel cost 10 % of the step.  (Without the
// launch attribute the instruction does nothing.)
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

}  // namespace cutb
