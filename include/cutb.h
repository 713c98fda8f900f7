/*
 * cutb.h -- C ABI of the B200 quantized-matmul backend for the CUT toolkit.
 *
 * One shared library (libcutb.so), plain pointers and sizes, no C++ or torch
 * types.  Every pointer named "device" is a CUDA device pointer on the current
 * device; `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * Calls enqueue work on `stream` and return without synchronising.  They
 * return CUTB_OK or an error code (never throw, never abort); a human-readable
 * message for the last error on the calling thread is kept in
 * cutb_last_error().  There is no CPU fallback: without a CUDA device every
 * compute entry point returns CUTB_ERR_CUDA.
 *
 * The entry points stand in for the kernels the reference reaches through
 * Dispatcher::encode -> ComputeInterface::encode -> cuLaunchKernel
 * (runtime/Dispatcher.cpp:18-75, core/backends/cuda/CudaCommandBuffer.cpp:128-245);
 * each declaration cites the reference interface it replaces.
 */
#ifndef CUTB_H
#define CUTB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CUTB_VERSION 100

/* Exported symbols: the library is built with hidden default visibility. */
#if defined(__GNUC__)
#define CUTB_API __attribute__((visibility("default")))
#else
#define CUTB_API
#endif

/* Status codes. */
enum {
  CUTB_OK = 0,
  CUTB_ERR_INVALID = 1,     /* bad shape, stride, pointer or enum value */
  CUTB_ERR_UNSUPPORTED = 2, /* valid request no kernel covers */
  CUTB_ERR_CUDA = 3,        /* a CUDA runtime call failed (no device, launch error) */
  CUTB_ERR_WORKSPACE = 4,   /* workspace missing or smaller than cutb_qmatmul_workspace_bytes() */
  CUTB_ERR_TIMEOUT = 5,     /* a bounded device-side wait ran out (read from the status word) */
  CUTB_ERR_RANGE = 6        /* an fp32 activation exceeded the fp16 operand range of the tensor-core GEMM (status word) */
};

/* GGUF block formats (interface/loader/gguf/gguf_types.hpp:109-150).  The matmul entry points
 * take the first three; cutb_dequant also takes the rest of the reference's DequantFormat set
 * (operators/impl/dequant/DequantOp.h:8-13): Q5_K (176-byte super-blocks), Q6_K (210-byte
 * super-blocks) and BF16 (2 bytes per element). */
enum { CUTB_Q8_0 = 0, CUTB_Q4_0 = 1, CUTB_Q4_K = 2, CUTB_Q5_K = 3, CUTB_Q6_K = 4, CUTB_BF16 = 5, CUTB_Q4_1 = 6, CUTB_Q5_0 = 7 };

/* Activation element types (core/api/include/ComputeCommon.h:107-113). */
enum { CUTB_F32 = 0, CUTB_F16 = 1 };

/* Weight layouts.
 *   CUTB_LAYOUT_GGUF_BLOCKS: N rows of native GGUF blocks along K, exactly the
 *     bytes GGUFReader::read_tensor_raw returns (gguf_reader.cpp:312-324).
 *   CUTB_LAYOUT_KN_PLANES: the reference's runtime layout -- values [K, N] int8
 *     (Q8) or [K, N/2] nibbles, low nibble = even n (Q4), plus fp16 scales
 *     [K/32, N]; with `affine` the scales plane has 2*K/32 rows, the lower half
 *     holding per-block mins (operators/impl/matmul/MatMulOp.cpp:309-329,
 *     MatMulQ4Common.cuh:126-153). */
enum { CUTB_LAYOUT_GGUF_BLOCKS = 0, CUTB_LAYOUT_KN_PLANES = 1 };

/* Fused epilogue selector = the reference's specialisation constants 1 and 2
 * (operators/impl/matmul/MatMulOp.cpp:484-498): 0 none, 1 unary, 2 binary with
 * the [M, N] operand D; `fusion_op` is the reference's OP_UNARY_* / OP_BINARY_*
 * code (operators/runtime/ComputeOpsShared.h:22-66, 118-186). */
enum { CUTB_FUSION_NONE = 0, CUTB_FUSION_UNARY = 1, CUTB_FUSION_BINARY = 2 };

/* Kernel variants of cutb_qmatmul (variant = -1 lets the library choose). */
enum {
  CUTB_VARIANT_AUTO = -1,
  CUTB_VARIANT_GENERIC = 0, /* any shape, SIMT, exact fp32 dequant + FMA */
  CUTB_VARIANT_GEMV_MMA = 1, /* decode: bulk-copy ring + int8 warp MMA, M <= 16 (fp16 A) / 8 (fp32 A); when forced, up to
                                four such row groups one after the other (M <= 64 / 32): faster than the GEMM on narrow
                                weights, which is what tuning rules are for */
  CUTB_VARIANT_GEMM_TC = 2, /* prefill: tcgen05 tensor-core GEMM, accumulators in tensor memory; its operands are fp16
                               (see the operand-range note at cutb_qmatmul_desc).  GGUF blocks (K % 256 == 0) and
                               CUTB_LAYOUT_KN_PLANES (K % 128 == 0; above four rows what CUTB_VARIANT_AUTO picks there) */
  CUTB_VARIANT_GEMV_PLANES = 3 /* decode over CUTB_LAYOUT_KN_PLANES (the reference's run-time layout), M <= 4: coalesced
                                  column groups, K split over warps and blocks */
};

/* Descriptor flags.
 *   CUTB_FLAG_NO_OVERLAP: by default the decode mat-vec is launched with
 *     programmatic stream serialization: its weight prefetch may begin while the
 *     previous kernel of the stream is still finishing, and it waits for that
 *     kernel to complete before it reads A or D or writes C.  This is only
 *     correct if the previous kernel does not write W (weights are constants of
 *     the model).  Set this flag to launch with plain stream ordering instead.
 *   CUTB_FLAG_ACT_16BIT: the decode mat-vec stages activations as 16-bit integers with one fp32
 *     scale per 32-k block.  fp32 activations are normally staged at two such levels (32 bits,
 *     fp32-accurate results); with this flag they are staged at one, which halves the tensor-core
 *     work and selects the fastest kernel shape for a single row.  The result then carries the
 *     error fp16 activations would (relative error of a dot product about 3e-5) but keeps the
 *     fp32 range, so large activations cannot overflow.  Ignored for fp16 activations and by the
 *     other variants.
 *   CUTB_FLAG_A_RMSNORM: the decode mat-vec normalises its activation rows while it stages them:
 *     A'[m, k] = A[m, k] * rsqrt(mean_k(A[m, k]^2) + a_norm_eps) * a_norm_weight[k], i.e. the
 *     RMSNorm that precedes every projection of a decoder layer (RMSNormOpNode,
 *     operators/impl/rmsnorm/RMSNormOp.cpp:7-76) without its own launch and round trip.  Only the
 *     CUTB_VARIANT_GEMV_MMA kernel implements it; other shapes return CUTB_ERR_UNSUPPORTED.
 *   CUTB_FLAG_GLU_PAIRS: gated projection in one launch.  W holds N rows in pairs -- row 2i of the
 *     gate matrix, row 2i + 1 of the up matrix -- and the output has N / 2 columns:
 *     C[m, i] = unary(fusion_op)(acc[m, 2i]) * acc[m, 2i + 1] (fusion_type CUTB_FUSION_UNARY; with
 *     SiLU this is the SwiGLU feed-forward the runner builds from matmulUnary + a multiply,
 *     interface/runner/llama/llama.cpp:2455-2470).  ldc >= N / 2.  The decode mat-vec (shapes that do
 *     not split K) and the tensor-core GEMM have it; anything else returns CUTB_ERR_UNSUPPORTED.
 *   CUTB_FLAG_STAGE_PER_CTA: from three activation rows up the decode mat-vec quantises its
 *     activations once per call, in a small launch of its own, into the workspace
 *     (cutb_qmatmul_workspace_bytes counts the room), and every block copies the result.  With this
 *     flag every block stages the activations itself, as it does for one or two rows: no staging
 *     scratch, slower for more than two rows.  The results are the same bit for bit. */
enum { CUTB_FLAG_NO_OVERLAP = 1, CUTB_FLAG_ACT_16BIT = 2, CUTB_FLAG_A_RMSNORM = 4, CUTB_FLAG_GLU_PAIRS = 8,
       CUTB_FLAG_STAGE_PER_CTA = 16 };

/*
 * C[M, N] = epilogue(A[M, K] * dequant(W)), fp32 accumulate, fp32 output.
 * Replaces the quantized MatMulOpNode dispatch: bindings (A, packedB, scalesB,
 * D, C) + push constants {M, K, N, strideA, strideB, strideC, scaleStride}
 * (operators/impl/matmul/MatMulOp.cpp:507-575, MatMulQ4Common.cuh:22-30).
 * Strides are in elements (bytes for W planes), as in the reference.
 *
 * Operand range.  The generic and the decode variants dequantise exactly and take fp32
 * activations at full range.  CUTB_VARIANT_GEMM_TC (what CUTB_VARIANT_AUTO picks above 8 fp32 /
 * 16 fp16 activation rows over GGUF blocks, and from 13 fp16 rows on weights of 16 M elements
 * and more) feeds the tensor cores fp16 operands, as the
 * reference's tensor-core variants do (MatMulQ4CoopMatTiled.cu:37-75): fp32 activations are
 * rounded to fp16 first, and a dequantised weight d * q (d * sc * q - dmin * m for Q4_K) is
 * rounded to fp16 too.  |A| above 65504 therefore becomes infinity, and the launch records
 * CUTB_ERR_RANGE in *status (the output then holds inf / NaN where such a value took part);
 * weight products below 6e-8 flush to zero.  Callers whose activations can exceed the fp16
 * range select CUTB_VARIANT_GENERIC, or scale A down and C up.  Accumulation and C are fp32.
 * Up to 128 activation rows the same variant runs a kernel of its own (tokens as the MMA's M
 * operand, K shared out over all SMs); it is launched with programmatic stream serialization
 * like the decode mat-vec (it waits for the previous kernel only before it reads A and before it
 * stores), which CUTB_FLAG_NO_OVERLAP switches off.
 */
typedef struct cutb_qmatmul_desc {
  int32_t format;      /* CUTB_Q8_0 / CUTB_Q4_0 / CUTB_Q4_K */
  int32_t layout;      /* CUTB_LAYOUT_* ; KN_PLANES supports Q8_0 and Q4_0 (+affine) */
  int32_t affine;      /* KN_PLANES + Q4 only: scales plane carries mins */
  int32_t a_dtype;     /* CUTB_F32 or CUTB_F16 */
  uint32_t M, K, N;
  const void *A;       /* device, [M, lda] */
  uint32_t lda;
  const void *W;       /* device: GGUF blocks, or the values plane */
  uint64_t W_bytes;    /* size of the W allocation, checked against the shape */
  const void *scales;  /* device, KN_PLANES only: fp16 [K/32 (x2 if affine), lds] */
  uint32_t ldb;        /* KN_PLANES: row stride of the values plane in bytes */
  uint32_t lds;        /* KN_PLANES: row stride of the scales plane in elements */
  float *C;            /* device, [M, ldc] */
  uint32_t ldc;
  const float *D;      /* device, [M, ldd]; only read when fusion_type == 2 */
  uint32_t ldd;
  int32_t fusion_type; /* CUTB_FUSION_* */
  int32_t fusion_op;   /* reference op code */
  int32_t variant;     /* CUTB_VARIANT_* */
  void *workspace;     /* device scratch, >= cutb_qmatmul_workspace_bytes(desc), 256-byte aligned; may be NULL if that is 0 */
  uint64_t workspace_bytes;
  int32_t *status;     /* optional device int: kernels store CUTB_ERR_TIMEOUT here if a bounded wait gives up,
                          CUTB_ERR_RANGE if an activation left the tensor-core GEMM's fp16 operand range */
  uint32_t flags;      /* CUTB_FLAG_* */
  const float *a_norm_weight; /* CUTB_FLAG_A_RMSNORM: device, [K] fp32 */
  float a_norm_eps;           /* CUTB_FLAG_A_RMSNORM */
} cutb_qmatmul_desc;

/* Scratch bytes cutb_qmatmul needs for this descriptor.  Never allocates.  What the variants keep there: the
 * decode mat-vec its staged activations (three rows and up) and split-K partial sums; the tensor-core GEMM the
 * fp16 copy of fp32 activations and, up to 128 activation rows, the partial tiles of weight tiles whose K is shared
 * by several blocks (summed in a fixed order by a second small kernel; without that room every weight tile goes
 * whole to one block, which is slower but needs nothing); with 512 rows and more on few weight rows and K >= 8192,
 * planes of partial sums of a K split (same rule: optional, faster with them). */
CUTB_API uint64_t cutb_qmatmul_workspace_bytes(const cutb_qmatmul_desc *desc);

/* Variant the library would run for this descriptor (resolves CUTB_VARIANT_AUTO);
 * negative on an invalid descriptor.  Mirrors the variant choice made in the
 * MatMulOpNode constructor (operators/impl/matmul/MatMulOp.cpp:335-380). */
CUTB_API int cutb_qmatmul_select_variant(const cutb_qmatmul_desc *desc);

CUTB_API int cutb_qmatmul(const cutb_qmatmul_desc *desc, void *stream);

/*
 * The decode mat-vec of cutb_qmatmul (variant CUTB_VARIANT_GEMV_MMA) for callers
 * that cannot allocate device memory -- servers that gave the whole GPU to their
 * own arena, plugins with a memory budget fixed at start-up.  It has no
 * counterpart in the reference.  desc->workspace is ignored: split-K partial
 * sums go to a 4 MiB array built into the library (resident in every GPU context
 * that loads it, until exit), so ksplit * M * N must not exceed 1,048,576
 * floats; larger shapes are rejected with CUTB_ERR_WORKSPACE and belong to
 * cutb_qmatmul with a caller-provided workspace.  It calls no allocating routine.
 * The first call on each device looks up the array's device address; make that
 * call outside any stream capture.  All calls share the one array and every
 * call overwrites the region it uses before reading it, so nothing needs
 * clearing between calls -- but two calls that overlap on the GPU (different
 * streams, or different host threads) race on it: serialise them.
 */
CUTB_API int cutb_qmatmul_decode_noalloc(const cutb_qmatmul_desc *desc, void *stream);

/*
 * Row-sharded decode mat-vec over several GPUs with the exchange step fused into the
 * kernel: rank r owns weight rows [n_offset, n_offset + desc->N) of a tensor of N_total rows,
 * computes its slice of the output and stores it into EVERY rank's full output
 * C_full[M, ldc_total] through peer-mapped device pointers (plain stores over NVLink; no
 * multicast object is involved).  It replaces "mat-vec, then all-gather of the slices".  The
 * reference has no counterpart (it offers a pipeline split with a host bounce only).
 *
 *   world         ranks (2 .. CUTB_MAX_PEERS); rank = this rank's index
 *   C_peers[q]    rank q's full output as mapped into THIS process (own buffer at [rank])
 *   flag_peers[q] rank q's arrival counter (one uint64, zero at the start, never reset)
 *   ldc_total     row stride of the full outputs (elements); n_offset: first column of the slice
 *
 * cutb_qmatmul_scatter: desc->C is not written.  The shape must take the mat-vec variant
 * (M <= 16 fp16 / 8 fp32 rows, K % 256 == 0), else CUTB_ERR_UNSUPPORTED; shapes that split K need
 * the workspace of cutb_qmatmul_workspace_bytes(desc) as usual (their reduction kernel scatters).
 * The stores are not yet published when it returns or when its kernel ends.
 *
 * cutb_peer_exchange is the step boundary, called by every rank once per step after the step's
 * scatter launches (any number of them, C_peers may differ per launch; only flag_peers, world
 * and rank are read here): a small kernel issues a system-scope fence and adds one to every
 * rank's counter, then polls this rank's own counter until all ranks have signalled the step or
 * about a second has passed (then *status = CUTB_ERR_TIMEOUT; nothing hangs).  The step number is
 * kept in *step_counter (a device uint64, zero at the start), so one captured launch serves
 * every replay of a CUDA graph.  Work enqueued after it on the stream sees every rank's slices.
 * Before an output buffer is scattered into again every rank must have consumed it (double
 * buffering by step parity is enough: no rank can be more than one step ahead of another).
 */
#define CUTB_MAX_PEERS 8
typedef struct cutb_peer_scatter {
  uint32_t world, rank;
  uint32_t ldc_total, n_offset;
  float *C_peers[CUTB_MAX_PEERS];
  uint64_t *flag_peers[CUTB_MAX_PEERS];
} cutb_peer_scatter;
CUTB_API int cutb_qmatmul_scatter(const cutb_qmatmul_desc *desc, const cutb_peer_scatter *peers, void *stream);
CUTB_API int cutb_peer_exchange(const cutb_peer_scatter *peers, uint64_t *step_counter, int *status, void *stream);

/*
 * Peer buffers of the fused exchange.  Every rank (one process per GPU) allocates ONE buffer for
 * its full outputs and its arrival counter, exports a handle, sends the 64 handle bytes to the
 * other ranks by any host channel, and opens theirs; the returned pointers are what
 * cutb_peer_scatter's C_peers / flag_peers are built from.  (CUDA IPC underneath: no multicast
 * object; the reference has no counterpart.)
 *
 *   cutb_peer_buffer_alloc   device memory on the current device, zero-filled, 256-byte aligned;
 *                            `handle` receives the 64 bytes to send
 *   cutb_peer_buffer_open    maps another rank's buffer into this process with the CURRENT device
 *                            as the accessing device (peer access is enabled by the runtime); a
 *                            handle exported by this same process is refused (use the pointer)
 *   cutb_peer_buffer_close   unmaps an opened buffer; cutb_peer_buffer_free frees an own buffer.
 *                            Close every mapping of a buffer before its owner frees it.
 * These calls allocate and synchronise: set-up and tear-down only, never inside a stream capture.
 */
#define CUTB_PEER_HANDLE_BYTES 64
CUTB_API int cutb_peer_buffer_alloc(uint64_t bytes, void **ptr, uint8_t handle[CUTB_PEER_HANDLE_BYTES]);
CUTB_API int cutb_peer_buffer_open(const uint8_t handle[CUTB_PEER_HANDLE_BYTES], void **ptr);
CUTB_API int cutb_peer_buffer_close(void *ptr);
CUTB_API int cutb_peer_buffer_free(void *ptr);

/*
 * Raw GGUF blocks -> fp32 [rows, cols] with row stride ldo (elements).
 * Replaces DequantOpNode's dispatch (operators/impl/dequant/DequantOp.cpp:7-61;
 * DequantQ4K.cu:6-50, DequantQ5K.cu, DequantQ6K.cu, DequantBF16.cu); Q8_0 and Q4_0
 * follow the loader's CPU dequantisers (interface/loader/gguf/gguf_reader.cpp:541-572,
 * 826-850).  Bit-exact with the loader's dequantisers for every format.  Q5_K and Q6_K
 * need cols % 256 == 0, as the reference's kernels do.
 */
CUTB_API int cutb_dequant(int format, const void *raw, uint64_t raw_bytes, float *out, uint32_t rows,
                 uint32_t cols, uint32_t ldo, void *stream);

/*
 * GGML-packed Q4_0 nibbles [N, stride_in bytes] -> [K, stride_out bytes] with
 * the low nibble holding even n.  Replaces TransposeQ4NibbleOpNode's dispatch
 * (operators/impl/q4transpose/TransposeQ4NibbleOp.cpp:7-59,
 * TransposeQ4Nibble.cu:36-61).  N even, K a multiple of 32.
 */
CUTB_API int cutb_transpose_q4(const void *in, void *out, uint32_t N, uint32_t K, uint32_t stride_in,
                      uint32_t stride_out, void *stream);

/* Library / device information. */
/*
 * Load-time repacks on the device, for callers that keep the reference's [K, N] plane layout
 * (the block kernels above need none of them).  Each is bit-exact with the CPU code it replaces.
 *
 * cutb_separate_blocks: Q8_0 / Q4_0 blocks of a row-major [rows, cols] tensor -> value plane
 *   (int8 [rows, cols], or GGML-packed nibbles [rows, cols / 2]) and f16 scale plane
 *   [rows, cols / 32], as GGUFReader::read_tensor_q8_separated / read_tensor_q4_separated return
 *   them (interface/loader/gguf/gguf_reader.cpp:389-501).  cols % 32 == 0.
 * cutb_transpose_2d: out[c * ldo + r] = in[r * ldi + c] for 1- or 2-byte elements (strides in
 *   elements): the runner's CPU transposes of the value and scale planes into the matmul's
 *   [K, N] orientation (interface/runner/llama/llama.cpp:934-1027).
 * cutb_requant_q4k_affine: Q4_K rows -> nibbles [K, ldp bytes] (low nibble = even n) and f16 planes
 *   [2 K / 32, lds]: rows [0, K / 32) = half(d sc), rows [K / 32, 2 K / 32) = half(8 d sc - dmin m),
 *   with the runner's float -> half rounding (llama.cpp:445-482, 573-619).  K % 256 == 0, N even;
 *   padding bytes of the outputs are not written.
 * cutb_quantize_rows_q8_0: n floats (n % 32 == 0, 16-byte aligned) -> int8 values and f16 scales,
 *   d = amax / 127, q = lround(x / d) (llama.cpp:488-505).
 * cutb_requant_q8_0_blocks: any format cutb_dequant takes -> Q8_0 GGUF blocks (34 bytes per 32
 *   weights, rows x cols / 32 of them), the exact dequantised values re-quantised as
 *   cutb_quantize_rows_q8_0 does.  This is the runner's load-time treatment of the formats its
 *   matmul does not take (Q4_1, Q5_0, Q5_K, Q6_K: llama.cpp:750-767, 934-1027), done on the device and
 *   straight into the block layout cutb_qmatmul reads; `out` 2-byte aligned, cols % 32 == 0.
 */
CUTB_API int cutb_separate_blocks(int format, const void *raw, uint64_t raw_bytes, void *values, void *scales, uint64_t rows,
                                  uint64_t cols, void *stream);
CUTB_API int cutb_transpose_2d(uint32_t elem_bytes, const void *in, void *out, uint32_t rows, uint32_t cols, uint64_t ldi,
                               uint64_t ldo, void *stream);
CUTB_API int cutb_requant_q4k_affine(const void *raw, uint64_t raw_bytes, void *packedT, void *scalesT, uint32_t N, uint32_t K,
                                     uint64_t ldp, uint64_t lds, void *stream);
CUTB_API int cutb_quantize_rows_q8_0(const float *x, void *values, void *scales, uint64_t n, void *stream);
CUTB_API int cutb_requant_q8_0_blocks(int format, const void *raw, uint64_t raw_bytes, void *out, uint64_t rows, uint32_t cols,
                                      void *stream);

/*
 * The operators on either side of the matmul in a decoder layer (first steps past the matmul
 * path; per token they move a few KB to a few hundred KB against the gigabytes of weights).
 *
 * cutb_rmsnorm: y[r, i] = x[r, i] * rsqrt(mean_i(x[r, i]^2) + eps) * weight[i] for `rows` rows of
 *   `dim` elements, row stride ldx elements, fp32 or fp16 (a_dtype codes), fp32 accumulation
 *   (RMSNormOpNode: operators/impl/rmsnorm/RMSNormOp.cpp:7-76, RMSNorm.cu:6-37; the reference
 *   pads the row stride to 4).
 * cutb_embedding: out[i, :] = table[indices[i], :], rows of pad4(dim) floats, 16-byte aligned
 *   (operators/impl/memory/Embedding.cu:18-35).  An index >= vocab writes zeros and sets *status
 *   to CUTB_ERR_INVALID instead of reading outside the table (the reference does not check).
 * cutb_embedding_col: out[i, d] = M[d, indices[i]] for a matrix kept in the matmul's [dim, vocab]
 *   orientation -- the embedding read out of a tied LM head (EmbeddingColOpNode:
 *   operators/impl/memory/MemoryOp.cpp:127-202, EmbeddingCol.cu:16-44).  format 0: fp16 matrix;
 *   format 1: int8 values with fp16 scales [dim / 32, vocab] (value * scale).  Strides in elements.
 *   An index >= vocab writes zeros and sets *status to CUTB_ERR_INVALID (the reference does not check).
 * cutb_embedding_blocks: the same lookup when the table is kept as raw GGUF blocks, one row of
 *   `cols` weights per token: out[i, :] = dequant(row indices[i]), bit-exact with cutb_dequant
 *   (every format of cutb_dequant).  It has no counterpart in the reference, whose runner either
 *   dequantises the whole table or gathers columns from the head (llama.cpp:1029-1060, 1425-1438).
 * cutb_argreduce: index of the maximum (is_max) or minimum of n floats, written as a float to
 *   out[0], with the reference's tie rule (the outcome of its 256-thread strided scan and
 *   shared-memory tree): among equal extremes the smallest bit-reversed (i mod 256) wins, then
 *   the smallest i (operators/impl/reduce/ReduceArg.cu:27-59).
 */
CUTB_API int cutb_rmsnorm(int dtype, const void *x, const void *weight, void *y, uint32_t rows, uint32_t dim, uint64_t ldx,
                          float eps, void *stream);
CUTB_API int cutb_embedding(const uint32_t *indices, const float *table, float *out, uint64_t n, uint32_t dim, uint32_t vocab,
                            int *status, void *stream);
CUTB_API int cutb_embedding_col(int format, const uint32_t *indices, const void *matrix, const void *scales, float *out, uint32_t n,
                                uint32_t dim, uint32_t vocab, uint32_t vocab_stride, uint32_t scale_stride, uint32_t out_stride,
                                int *status, void *stream);
CUTB_API int cutb_embedding_blocks(int format, const uint32_t *indices, const void *raw, float *out, uint32_t n, uint32_t rows,
                                   uint32_t cols, uint32_t ldo, int *status, void *stream);
CUTB_API int cutb_argreduce(int is_max, const float *values, float *out, uint32_t n, void *stream);

/*
 * Decode-step attention for one token.  `params` is the reference's two-word device buffer
 * {pos, seqLen} (interface/runner/llama/llama.cpp:2087-2094), read by the kernels, so a recorded
 * step replays for every token.  Caches are [max_seq][ld] elements (ld >= n_kv_heads * head_dim,
 * the reference pads it to 4), kv_dtype CUTB_F32 or CUTB_F16; head_dim even and <= 128.
 *
 * cutb_rope_kv_write: half-split rotary embedding of q[q_dim] and k[kv_dim] with the tables
 *   cos/sin[max_seq][head_dim / 2] at row pos; writes q_out[q_dim], the roped k into
 *   k_cache[pos] and v into v_cache[pos] (FusedRoPEKVWriteOpNode's dispatch,
 *   operators/impl/attention/FusedRoPEKVWrite.cu:13-75).  pos >= max_seq writes nothing and sets
 *   *status to CUTB_ERR_INVALID (the reference does not check).
 * cutb_attention_decode: out[h] = softmax(scale * q[h] . K[0..seqLen)) . V[0..seqLen) per query
 *   head, head h reading KV head h / (n_heads / n_kv_heads) (AttentionOpNode's dispatch,
 *   operators/impl/attention/Attention.cu:31-108).  n_heads / n_kv_heads <= 8, max_seq <= 32768.
 *   seqLen > max_seq is clamped and reported through *status.  `workspace` holds
 *   cutb_attention_workspace_bytes() bytes; its first 256 bytes must be zero before the first
 *   call and are left zero by every call (launches sharing a workspace must not overlap).
 * cutb_rope_attention_decode: cutb_rope_kv_write followed by cutb_attention_decode as ONE launch
 *   where the cluster kernel applies (head_dim % 32 == 0, 1 / 2 / 4 / 8 query heads per KV head,
 *   slices that fit in shared memory): every slice rotates its own copy of q, the slice that owns
 *   row pos takes the rotated k and v straight into its tile and the first slice stores them to
 *   the caches.  Other shapes run the two kernels back to back.  Same results as the two calls
 *   (cache rows bit-exact); the rotated q is not returned.  q, k, v must not alias the caches.
 */
CUTB_API int cutb_rope_kv_write(int kv_dtype, const float *q, const float *k, const float *v, const uint32_t *params,
                                const float *cos_table, const float *sin_table, void *k_cache, void *v_cache, float *q_out,
                                uint32_t q_dim, uint32_t kv_dim, uint32_t head_dim, uint64_t ld, uint32_t max_seq, int *status,
                                void *stream);
CUTB_API uint64_t cutb_attention_workspace_bytes(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_seq);
/*
 * Prefill (a batch of prompt tokens) over the same caches.  positions[i] is token i's cache row.
 * cutb_batched_kv_write: k_cache[positions[i]] = RoPE(k_in[i]), v_cache[positions[i]] = v_in[i]; rows of
 *   k_in / v_in are k_stride / v_stride elements apart, so they may be columns of a fused QKV matrix
 *   (BatchedKVCacheWriteOpNode's dispatch, operators/impl/attention/BatchedKVCacheWrite.cu:33-62).
 * cutb_batched_attention: out[i] = attention of RoPE(q_in[i]) over cache rows [0, positions[i]], one block
 *   per (KV head, group of consecutive tokens) (operators/impl/attention/BatchedAttentionReadCache.cu).  A block
 *   walks its tokens' range in chunks of 512 rows with a running maximum and exp-sum, so positions[i] < max_seq is
 *   the only limit (a position past the cache is reported through `status`, never read).  Call after the cache write.
 *   With an fp16 cache, head_dim 64 or 128, 16-byte aligned cache rows and 16 tokens or more the products run on the
 *   tensor cores (64 tokens of a query head per block, K / V tiles of 64 rows, online softmax): the rotated queries
 *   and the probabilities are rounded to fp16 there, sums stay fp32 -- within about 1e-3 of the output's magnitude of
 *   the fp32 arithmetic of the other shapes.
 * cutb_glu_pairs: out[r, i] = unary(op)(in[r, 2i]) * in[r, 2i + 1] (ldi even, 8-byte aligned `in`): the
 *   gated activation over a prefill GEMM whose weight rows are stored in (gate, up) pairs.
 */
CUTB_API int cutb_batched_kv_write(int kv_dtype, const float *k_in, const float *v_in, uint32_t k_stride, uint32_t v_stride,
                                   const uint32_t *positions, const float *cos_table, const float *sin_table, void *k_cache,
                                   void *v_cache, uint32_t n_tokens, uint32_t kv_dim, uint32_t head_dim, uint64_t ld, uint32_t max_seq,
                                   int *status, void *stream);
CUTB_API int cutb_batched_attention(int kv_dtype, const float *q_in, uint32_t q_stride, const void *k_cache, const void *v_cache,
                                    const uint32_t *positions, const float *cos_table, const float *sin_table, float *out,
                                    uint32_t out_stride, uint32_t n_tokens, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                                    uint64_t ld, uint32_t max_seq, float scale, int *status, void *stream);
/*
 * n device-to-device byte copies in one launch (no counterpart in the reference).  `table` holds n ranges
 * {src, dst, bytes}; src and dst 16-byte aligned, ranges must not overlap each other.  The table is read by the
 * kernel: device memory or host-mapped pinned memory (pass its device address), unchanged until the launch has run.
 * A backend scatters one coalesced upload into its tensors with it, and gathers a step's results for one download.
 */
typedef struct cutb_copy_range {
  const void *src;
  void *dst;
  uint64_t bytes;
} cutb_copy_range;
CUTB_API int cutb_copy_batch(const cutb_copy_range *table, uint32_t n, uint64_t max_bytes, void *stream);

CUTB_API int cutb_glu_pairs(const float *in, float *out, uint32_t rows, uint32_t cols_out, uint64_t ldi, uint64_t ldo, int unary_op,
                            void *stream);
CUTB_API int cutb_rope_attention_decode(int kv_dtype, const float *q, const float *k, const float *v, const uint32_t *params,
                                        const float *cos_table, const float *sin_table, void *k_cache, void *v_cache, float *out,
                                        uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint64_t ld, uint32_t max_seq,
                                        float scale, void *workspace, uint64_t workspace_bytes, int *status, void *stream);
CUTB_API int cutb_attention_decode(int kv_dtype, const float *q, const void *k_cache, const void *v_cache, const uint32_t *params,
                                   float *out, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint64_t ld,
                                   uint32_t max_seq, float scale, void *workspace, uint64_t workspace_bytes, int *status,
                                   void *stream);

CUTB_API int cutb_version(void);
CUTB_API const char *cutb_status_string(int status);
CUTB_API const char *cutb_last_error(void);
/* Number of streaming multiprocessors of the current device, or -1. */
CUTB_API int cutb_device_sm_count(void);
CUTB_API const char *cutb_variant_name(int variant);

#ifdef __cplusplus
}
#endif
#endif /* CUTB_H */
