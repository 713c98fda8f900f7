// extern "C" entry points of libcutb.so: argument validation, variant choice,
// launch.  No allocation, no synchronisation, no CPU fallback.
#include <string.h>

#include "common.cuh"
#include "kernels.h"

namespace cutb {
const char *last_error();

namespace {

int validate(const cutb_qmatmul_desc *d) {
  if (!d) {
    set_last_error("qmatmul: null descriptor");
    return CUTB_ERR_INVALID;
  }
  if (d->format < CUTB_Q8_0 || d->format > CUTB_Q4_K) {
    set_last_error("qmatmul: unknown format %d", d->format);
    return CUTB_ERR_INVALID;
  }
  if (d->layout != CUTB_LAYOUT_GGUF_BLOCKS && d->layout != CUTB_LAYOUT_KN_PLANES) {
    set_last_error("qmatmul: unknown layout %d", d->layout);
    return CUTB_ERR_INVALID;
  }
  if (d->a_dtype != CUTB_F32 && d->a_dtype != CUTB_F16) {
    set_last_error("qmatmul: unknown activation dtype %d", d->a_dtype);
    return CUTB_ERR_INVALID;
  }
  if (d->M == 0 || d->K == 0 || d->N == 0) {
    set_last_error("qmatmul: empty shape M=%u K=%u N=%u", d->M, d->K, d->N);
    return CUTB_ERR_INVALID;
  }
  if (!d->A || !d->W || !d->C) {
    set_last_error("qmatmul: null A, W or C");
    return CUTB_ERR_INVALID;
  }
  const bool glu = (d->flags & CUTB_FLAG_GLU_PAIRS) != 0;
  if (glu && (d->N % 2 != 0 || d->fusion_type != CUTB_FUSION_UNARY)) {
    set_last_error("qmatmul: CUTB_FLAG_GLU_PAIRS needs an even N and a unary fusion (the gate's activation)");
    return CUTB_ERR_INVALID;
  }
  if (d->lda < d->K || d->ldc < (glu ? d->N / 2 : d->N)) {
    set_last_error("qmatmul: lda (%u) < K (%u) or ldc (%u) < N (%u)", d->lda, d->K, d->ldc, d->N);
    return CUTB_ERR_INVALID;
  }
  if (d->fusion_type < CUTB_FUSION_NONE || d->fusion_type > CUTB_FUSION_BINARY) {
    set_last_error("qmatmul: unknown fusion type %d", d->fusion_type);
    return CUTB_ERR_INVALID;
  }
  if (d->fusion_type == CUTB_FUSION_BINARY && (!d->D || d->ldd < d->N)) {
    set_last_error("qmatmul: binary fusion needs D with ldd >= N");
    return CUTB_ERR_INVALID;
  }
  if (d->layout == CUTB_LAYOUT_GGUF_BLOCKS) {
    if (d->K % block_elems(d->format) != 0) {
      set_last_error("qmatmul: K=%u is not a multiple of the block size %u", d->K, block_elems(d->format));
      return CUTB_ERR_INVALID;
    }
    const uint64_t need = (uint64_t)d->N * row_bytes(d->format, d->K);
    if (d->W_bytes < need) {
      set_last_error("qmatmul: W holds %llu bytes, shape needs %llu", (unsigned long long)d->W_bytes, (unsigned long long)need);
      return CUTB_ERR_INVALID;
    }
    if (d->affine) {
      set_last_error("qmatmul: affine applies to the plane layout only");
      return CUTB_ERR_INVALID;
    }
  } else {
    if (d->format == CUTB_Q4_K) {
      set_last_error("qmatmul: the plane layout carries Q8 or Q4 (+affine), not Q4_K super-blocks");
      return CUTB_ERR_INVALID;
    }
    if (!d->scales) {
      set_last_error("qmatmul: plane layout needs a scales plane");
      return CUTB_ERR_INVALID;
    }
    const uint32_t vals_cols = d->format == CUTB_Q4_0 ? (d->N + 1) / 2 : d->N;
    if (d->ldb < vals_cols || d->lds < d->N) {
      set_last_error("qmatmul: ldb (%u) or lds (%u) too small for N=%u", d->ldb, d->lds, d->N);
      return CUTB_ERR_INVALID;
    }
    if (d->format == CUTB_Q4_0 && (d->N & 1)) {
      set_last_error("qmatmul: Q4 plane layout needs an even N");
      return CUTB_ERR_INVALID;
    }
    if (d->affine && d->format != CUTB_Q4_0) {
      set_last_error("qmatmul: affine applies to Q4 only");
      return CUTB_ERR_INVALID;
    }
    const uint64_t need = (uint64_t)(d->K - 1) * d->ldb + vals_cols;
    if (d->W_bytes < need) {
      set_last_error("qmatmul: W holds %llu bytes, shape needs %llu", (unsigned long long)d->W_bytes, (unsigned long long)need);
      return CUTB_ERR_INVALID;
    }
  }
  if (d->variant < CUTB_VARIANT_AUTO || d->variant > CUTB_VARIANT_GEMV_PLANES) {
    set_last_error("qmatmul: unknown variant %d", d->variant);
    return CUTB_ERR_INVALID;
  }
  return CUTB_OK;
}

// Decode shapes go to the bulk-copy MMA mat-vec, prefill shapes to the
// tensor-core GEMM, everything else to the SIMT kernel.  The reference makes
// the same split on M (operators/impl/matmul/MatMulOp.cpp:335-380).
int select(const cutb_qmatmul_desc &d) {
  if (d.variant != CUTB_VARIANT_AUTO) return d.variant;
  if (d.layout == CUTB_LAYOUT_GGUF_BLOCKS) {
    if (qgemv_blocks_supported(d)) {
      // 13 to 16 fp16 rows need the mat-vec's fourth column tile; from 16 M weights up the tensor-core GEMM for few
      // tokens is faster there (16 rows: 4096 x 4096 15.0 against 11.2 us, 11008 x 4096 28.0 against 22.1 us; at
      // 2048 x 2048 the mat-vec wins, 6.1 against 7.5 us).  The fused RMSNorm exists in the mat-vec only.
      const bool matvec_only = d.flags & CUTB_FLAG_A_RMSNORM;
      if (d.a_dtype == CUTB_F16 && d.M >= 13 && (uint64_t)d.K * d.N >= (1ull << 24) && !matvec_only && qgemm_tc_supported(d))
        return CUTB_VARIANT_GEMM_TC;
      return CUTB_VARIANT_GEMV_MMA;
    }
    if (qgemm_tc_supported(d)) return CUTB_VARIANT_GEMM_TC;
  } else if (qgemv_planes_supported(d)) {
    return CUTB_VARIANT_GEMV_PLANES;
  } else if (qgemm_tc_supported(d)) {
    return CUTB_VARIANT_GEMM_TC;  // prefill over the planes: the tensor-core GEMM with plane converters
  }
  return CUTB_VARIANT_GENERIC;
}

}  // namespace

int check_qmatmul_desc(const cutb_qmatmul_desc *d) { return validate(d); }

}  // namespace cutb

using namespace cutb;

extern "C" {

int cutb_version(void) { return CUTB_VERSION; }

const char *cutb_status_string(int status) {
  switch (status) {
    case CUTB_OK: return "ok";
    case CUTB_ERR_INVALID: return "invalid argument";
    case CUTB_ERR_UNSUPPORTED: return "unsupported request";
    case CUTB_ERR_CUDA: return "CUDA error";
    case CUTB_ERR_WORKSPACE: return "workspace missing or too small";
    case CUTB_ERR_TIMEOUT: return "device-side wait timed out";
    case CUTB_ERR_RANGE: return "activation outside the fp16 operand range";
    default: return "unknown status";
  }
}

const char *cutb_last_error(void) { return cutb::last_error(); }

const char *cutb_variant_name(int variant) {
  switch (variant) {
    case CUTB_VARIANT_GENERIC: return "QMatMulGeneric";
    case CUTB_VARIANT_GEMV_MMA: return "QGemvBulkMma";
    case CUTB_VARIANT_GEMM_TC: return "QGemmTcgen05";
    case CUTB_VARIANT_GEMV_PLANES: return "QGemvPlanes";
    default: return "Unknown";
  }
}

int cutb_device_sm_count(void) {
  DeviceInfo di;
  if (get_device_info(&di) != CUTB_OK) return -1;
  return di.sm_count;
}

int cutb_qmatmul_select_variant(const cutb_qmatmul_desc *desc) {
  if (validate(desc) != CUTB_OK) return -1;
  return select(*desc);
}

uint64_t cutb_qmatmul_workspace_bytes(const cutb_qmatmul_desc *desc) {
  if (validate(desc) != CUTB_OK) return 0;
  const int v = select(*desc);
  if (v == CUTB_VARIANT_GEMV_MMA) return qgemv_blocks_workspace(*desc);
  if (v == CUTB_VARIANT_GEMM_TC) return qgemm_tc_workspace(*desc);
  if (v == CUTB_VARIANT_GEMV_PLANES) return qgemv_planes_workspace(*desc);
  return 0;
}

int cutb_qmatmul(const cutb_qmatmul_desc *desc, void *stream) {
  if (int rc = validate(desc)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int v = select(*desc);
  if ((desc->flags & CUTB_FLAG_GLU_PAIRS) && v != CUTB_VARIANT_GEMV_MMA && v != CUTB_VARIANT_GEMM_TC) {
    // (the mat-vec launcher refuses shapes that split K; the tensor-core GEMMs take every shape they support)
    set_last_error("qmatmul: paired gate/up rows exist in the decode mat-vec and the tensor-core GEMM only");
    return CUTB_ERR_UNSUPPORTED;
  }
  if (desc->flags & CUTB_FLAG_A_RMSNORM) {
    if (!desc->a_norm_weight) {
      set_last_error("qmatmul: CUTB_FLAG_A_RMSNORM without a_norm_weight");
      return CUTB_ERR_INVALID;
    }
    if (v != CUTB_VARIANT_GEMV_MMA) {
      set_last_error("qmatmul: the fused RMSNorm exists in the decode mat-vec only (variant %s was selected)", cutb_variant_name(v));
      return CUTB_ERR_UNSUPPORTED;
    }
  }
  switch (v) {
    case CUTB_VARIANT_GEMV_MMA:
      if (!qgemv_blocks_supported(*desc) && !qgemv_blocks_supported_in_groups(*desc)) {
        set_last_error("qmatmul: variant %s needs GGUF blocks, K %% 256 == 0, 16-byte aligned W and M <= 64 (fp16) / 32 (fp32) "
                       "(beyond 16 / 8 rows in groups, without paired rows)",
                       cutb_variant_name(v));
        return CUTB_ERR_UNSUPPORTED;
      }
      return qgemv_blocks_launch(*desc, s);
    case CUTB_VARIANT_GEMM_TC:
      if (!qgemm_tc_supported(*desc)) {
        set_last_error("qmatmul: variant %s does not cover this shape/layout", cutb_variant_name(v));
        return CUTB_ERR_UNSUPPORTED;
      }
      return qgemm_tc_launch(*desc, s);
    case CUTB_VARIANT_GEMV_PLANES:
      if (!qgemv_planes_supported(*desc)) {
        set_last_error("qmatmul: variant %s needs the [K, N] plane layout (Q8 or Q4), M <= 4 and strides padded to 4", cutb_variant_name(v));
        return CUTB_ERR_UNSUPPORTED;
      }
      return qgemv_planes_launch(*desc, s);
    default:
      return qmatmul_generic_launch(*desc, s);
  }
}

namespace {
int check_peers(const cutb_peer_scatter *peers, const char *who) {
  if (!peers || peers->world < 2 || peers->world > CUTB_MAX_PEERS || peers->rank >= peers->world) {
    set_last_error("%s: world must be 2..%d and rank < world", who, CUTB_MAX_PEERS);
    return CUTB_ERR_INVALID;
  }
  for (uint32_t q = 0; q < peers->world; ++q)
    if (!peers->C_peers[q] || !peers->flag_peers[q] || reinterpret_cast<uintptr_t>(peers->flag_peers[q]) % 8 != 0) {
      set_last_error("%s: rank %u's output or counter pointer is null or misaligned", who, q);
      return CUTB_ERR_INVALID;
    }
  return CUTB_OK;
}
}  // namespace

int cutb_qmatmul_scatter(const cutb_qmatmul_desc *desc, const cutb_peer_scatter *peers, void *stream) {
  if (int rc = validate(desc)) return rc;
  if (int rc = check_peers(peers, "qmatmul_scatter")) return rc;
  if ((uint64_t)peers->n_offset + desc->N > peers->ldc_total) {
    set_last_error("qmatmul_scatter: slice [%u, %u) exceeds the row stride %u of the full output", peers->n_offset,
                   peers->n_offset + desc->N, peers->ldc_total);
    return CUTB_ERR_INVALID;
  }
  cutb_qmatmul_desc d = *desc;
  d.variant = CUTB_VARIANT_GEMV_MMA;
  if (!qgemv_blocks_supported(d)) {
    set_last_error("qmatmul_scatter: needs GGUF blocks, K %% 256 == 0, 16-byte aligned W and M <= 16 (fp16) / 8 (fp32)");
    return CUTB_ERR_UNSUPPORTED;
  }
  return qgemv_blocks_launch(d, reinterpret_cast<cudaStream_t>(stream), peers);
}

int cutb_peer_buffer_alloc(uint64_t bytes, void **ptr, uint8_t handle[CUTB_PEER_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == CUTB_PEER_HANDLE_BYTES, "handle size");
  if (!ptr || !handle || bytes == 0) {
    set_last_error("peer_buffer_alloc: null argument or zero size");
    return CUTB_ERR_INVALID;
  }
  void *p = nullptr;
  CUTB_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "cudaIpcGetMemHandle");
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return CUTB_OK;
}

int cutb_peer_buffer_open(const uint8_t handle[CUTB_PEER_HANDLE_BYTES], void **ptr) {
  if (!ptr || !handle) {
    set_last_error("peer_buffer_open: null argument");
    return CUTB_ERR_INVALID;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void *p = nullptr;
  CUTB_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return CUTB_OK;
}

int cutb_peer_buffer_close(void *ptr) {
  if (!ptr) return CUTB_OK;
  CUTB_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return CUTB_OK;
}

int cutb_peer_buffer_free(void *ptr) {
  if (!ptr) return CUTB_OK;
  CUTB_CUDA_TRY(cudaFree(ptr));
  return CUTB_OK;
}

int cutb_peer_exchange(const cutb_peer_scatter *peers, uint64_t *step_counter, int *status, void *stream) {
  if (int rc = check_peers(peers, "peer_exchange")) return rc;
  if (!step_counter || reinterpret_cast<uintptr_t>(step_counter) % 8 != 0) {
    set_last_error("peer_exchange: null or misaligned step counter");
    return CUTB_ERR_INVALID;
  }
  return peer_exchange_launch(*peers, step_counter, status, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_separate_blocks(int format, const void *raw, uint64_t raw_bytes, void *values, void *scales, uint64_t rows, uint64_t cols,
                         void *stream) {
  if (format != CUTB_Q8_0 && format != CUTB_Q4_0) {
    set_last_error("separate_blocks: format must be Q8_0 or Q4_0");
    return CUTB_ERR_INVALID;
  }
  if (rows == 0 || cols == 0) return CUTB_OK;
  if (!raw || !values || !scales || cols % 32 != 0 || reinterpret_cast<uintptr_t>(raw) % 2 || reinterpret_cast<uintptr_t>(values) % 2 ||
      reinterpret_cast<uintptr_t>(scales) % 2) {
    set_last_error("separate_blocks: null or odd pointer, or cols %% 32 != 0");
    return CUTB_ERR_INVALID;
  }
  if (raw_bytes < rows * (cols / 32) * block_bytes(format)) {
    set_last_error("separate_blocks: %llu raw bytes for %llu x %llu", (unsigned long long)raw_bytes, (unsigned long long)rows,
                   (unsigned long long)cols);
    return CUTB_ERR_INVALID;
  }
  return separate_launch(format, raw, values, scales, rows, cols, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_transpose_2d(uint32_t elem_bytes, const void *in, void *out, uint32_t rows, uint32_t cols, uint64_t ldi, uint64_t ldo,
                      void *stream) {
  if (elem_bytes != 1 && elem_bytes != 2) {
    set_last_error("transpose_2d: element size must be 1 or 2 bytes");
    return CUTB_ERR_INVALID;
  }
  if (rows == 0 || cols == 0) return CUTB_OK;
  if (!in || !out || ldi < cols || ldo < rows || reinterpret_cast<uintptr_t>(in) % elem_bytes || reinterpret_cast<uintptr_t>(out) % elem_bytes) {
    set_last_error("transpose_2d: null or misaligned pointer, or a stride shorter than the row");
    return CUTB_ERR_INVALID;
  }
  return transpose_launch(elem_bytes, in, out, rows, cols, ldi, ldo, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_requant_q4k_affine(const void *raw, uint64_t raw_bytes, void *packedT, void *scalesT, uint32_t N, uint32_t K, uint64_t ldp,
                            uint64_t lds, void *stream) {
  if (K % 256 != 0 || N % 2 != 0) {  // the reference declines these shapes too (llama.cpp:576-578)
    set_last_error("requant_q4k_affine: needs K %% 256 == 0 and even N (K=%u N=%u)", K, N);
    return CUTB_ERR_UNSUPPORTED;
  }
  if (N == 0 || K == 0) return CUTB_OK;
  if (!raw || !packedT || !scalesT || reinterpret_cast<uintptr_t>(raw) % 4 || reinterpret_cast<uintptr_t>(scalesT) % 2 || ldp < N / 2 ||
      lds < N || raw_bytes < (uint64_t)N * (K / 256) * 144) {
    set_last_error("requant_q4k_affine: null or misaligned pointer, short stride or short input");
    return CUTB_ERR_INVALID;
  }
  return requant_q4k_affine_launch(raw, packedT, scalesT, N, K, ldp, lds, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_quantize_rows_q8_0(const float *x, void *values, void *scales, uint64_t n, void *stream) {
  if (n == 0) return CUTB_OK;
  if (!x || !values || !scales || n % 32 != 0 || reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(values) % 16 ||
      reinterpret_cast<uintptr_t>(scales) % 2) {
    set_last_error("quantize_rows_q8_0: null or misaligned pointer, or n %% 32 != 0");
    return CUTB_ERR_INVALID;
  }
  return quantize_rows_q8_0_launch(x, values, scales, n, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_requant_q8_0_blocks(int format, const void *raw, uint64_t raw_bytes, void *out, uint64_t rows, uint32_t cols, void *stream) {
  if (rows == 0 || cols == 0) return CUTB_OK;
  if (format < CUTB_Q8_0 || format > CUTB_Q5_0) {
    set_last_error("requant_q8_0_blocks: unknown block format %d", format);
    return CUTB_ERR_INVALID;
  }
  const uint32_t be = block_elems(format);
  if (!raw || !out || cols % 32 != 0 || cols % be != 0 || reinterpret_cast<uintptr_t>(out) % 2 != 0) {
    set_last_error("requant_q8_0_blocks: null pointer, misaligned output, or cols (%u) not a whole number of blocks", cols);
    return CUTB_ERR_INVALID;
  }
  if (raw_bytes < rows * row_bytes(format, cols)) {
    set_last_error("requant_q8_0_blocks: %llu raw bytes given, %llu needed", (unsigned long long)raw_bytes,
                   (unsigned long long)(rows * row_bytes(format, cols)));
    return CUTB_ERR_INVALID;
  }
  return requant_q8_0_blocks_launch(format, raw, out, rows, cols, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_rmsnorm(int dtype, const void *x, const void *weight, void *y, uint32_t rows, uint32_t dim, uint64_t ldx, float eps,
                 void *stream) {
  if (dtype != CUTB_F32 && dtype != CUTB_F16) {
    set_last_error("rmsnorm: dtype must be fp32 or fp16");
    return CUTB_ERR_INVALID;
  }
  if (rows == 0 || dim == 0) return CUTB_OK;
  if (!x || !weight || !y || ldx < dim) {
    set_last_error("rmsnorm: null pointer or row stride shorter than the row");
    return CUTB_ERR_INVALID;
  }
  return rmsnorm_launch(dtype, x, weight, y, rows, dim, ldx, eps, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_embedding(const uint32_t *indices, const float *table, float *out, uint64_t n, uint32_t dim, uint32_t vocab, int *status,
                   void *stream) {
  if (n == 0 || dim == 0) return CUTB_OK;
  if (!indices || !table || !out || reinterpret_cast<uintptr_t>(table) % 16 || reinterpret_cast<uintptr_t>(out) % 16) {
    set_last_error("embedding: null pointer, or table / output not 16-byte aligned");
    return CUTB_ERR_INVALID;
  }
  return embedding_launch(indices, table, out, n, dim, vocab, status, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_embedding_col(int format, const uint32_t *indices, const void *matrix, const void *scales, float *out, uint32_t n,
                       uint32_t dim, uint32_t vocab, uint32_t vocab_stride, uint32_t scale_stride, uint32_t out_stride, int *status,
                       void *stream) {
  if (n == 0 || dim == 0) return CUTB_OK;
  if (format != 0 && format != 1) {
    set_last_error("embedding_col: format must be 0 (fp16 matrix) or 1 (int8 values + fp16 scales)");
    return CUTB_ERR_INVALID;
  }
  if (!indices || !matrix || !out || (format == 1 && !scales)) {
    set_last_error("embedding_col: null pointer");
    return CUTB_ERR_INVALID;
  }
  if (vocab_stride < vocab || out_stride < dim || (format == 1 && scale_stride < vocab) ||
      (format == 0 && reinterpret_cast<uintptr_t>(matrix) % 2) || (format == 1 && reinterpret_cast<uintptr_t>(scales) % 2)) {
    set_last_error("embedding_col: a stride is shorter than its row, or an fp16 pointer is misaligned");
    return CUTB_ERR_INVALID;
  }
  return embedding_col_launch(format, indices, matrix, scales, out, n, dim, vocab, vocab_stride, scale_stride, out_stride, status,
                              reinterpret_cast<cudaStream_t>(stream));
}

int cutb_embedding_blocks(int format, const uint32_t *indices, const void *raw, float *out, uint32_t n, uint32_t rows, uint32_t cols,
                          uint32_t ldo, int *status, void *stream) {
  if (n == 0 || cols == 0) return CUTB_OK;
  if (format < CUTB_Q8_0 || format > CUTB_Q5_0) {
    set_last_error("embedding_blocks: unknown block format %d", format);
    return CUTB_ERR_INVALID;
  }
  if (!indices || !raw || !out || ldo < cols || cols % block_elems(format) != 0) {
    set_last_error("embedding_blocks: null pointer, ldo < cols, or cols not a whole number of blocks");
    return CUTB_ERR_INVALID;
  }
  return dequant_gather_launch(format, indices, raw, out, n, rows, cols, ldo, status, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_argreduce(int is_max, const float *values, float *out, uint32_t n, void *stream) {
  if (!out || (n && !values)) {
    set_last_error("argreduce: null pointer");
    return CUTB_ERR_INVALID;
  }
  return argreduce_launch(is_max, values, out, n, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_rope_kv_write(int kv_dtype, const float *q, const float *k, const float *v, const uint32_t *params, const float *cos_table,
                       const float *sin_table, void *k_cache, void *v_cache, float *q_out, uint32_t q_dim, uint32_t kv_dim,
                       uint32_t head_dim, uint64_t ld, uint32_t max_seq, int *status, void *stream) {
  if (kv_dtype != CUTB_F32 && kv_dtype != CUTB_F16) {
    set_last_error("rope_kv_write: cache dtype must be fp32 or fp16");
    return CUTB_ERR_INVALID;
  }
  if (!q || !k || !v || !params || !cos_table || !sin_table || !k_cache || !v_cache || !q_out) {
    set_last_error("rope_kv_write: null pointer");
    return CUTB_ERR_INVALID;
  }
  if (head_dim == 0 || head_dim % 2 || q_dim % head_dim || kv_dim % head_dim || ld < kv_dim || max_seq == 0) {
    set_last_error("rope_kv_write: head_dim must be even and divide q_dim and kv_dim; ld >= kv_dim; max_seq > 0");
    return CUTB_ERR_INVALID;
  }
  return rope_kv_write_launch(kv_dtype, q, k, v, params, cos_table, sin_table, k_cache, v_cache, q_out, q_dim, kv_dim, head_dim, ld,
                              max_seq, status, reinterpret_cast<cudaStream_t>(stream));
}

uint64_t cutb_attention_workspace_bytes(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_seq) {
  return attention_workspace_bytes(n_heads, n_kv_heads, head_dim, max_seq);
}

int cutb_attention_decode(int kv_dtype, const float *q, const void *k_cache, const void *v_cache, const uint32_t *params, float *out,
                          uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint64_t ld, uint32_t max_seq, float scale,
                          void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
  if (kv_dtype != CUTB_F32 && kv_dtype != CUTB_F16) {
    set_last_error("attention: cache dtype must be fp32 or fp16");
    return CUTB_ERR_INVALID;
  }
  if (!q || !k_cache || !v_cache || !params || !out || !workspace) {
    set_last_error("attention: null pointer");
    return CUTB_ERR_INVALID;
  }
  if (n_heads == 0 || n_kv_heads == 0 || n_heads % n_kv_heads || n_heads / n_kv_heads > 8 || head_dim == 0 || head_dim > 128 ||
      ld < (uint64_t)n_kv_heads * head_dim || max_seq == 0) {
    set_last_error("attention: need n_heads = n_kv_heads * (1..8), head_dim in 1..128, ld >= n_kv_heads * head_dim, max_seq > 0");
    return CUTB_ERR_INVALID;
  }
  if (reinterpret_cast<uintptr_t>(workspace) % 16 || workspace_bytes < attention_workspace_bytes(n_heads, n_kv_heads, head_dim, max_seq)) {
    set_last_error("attention: workspace must be 16-byte aligned and hold %llu bytes",
                   (unsigned long long)attention_workspace_bytes(n_heads, n_kv_heads, head_dim, max_seq));
    return CUTB_ERR_INVALID;
  }
  return attention_decode_launch(kv_dtype, q, k_cache, v_cache, params, out, n_heads, n_kv_heads, head_dim, ld, max_seq, scale,
                                 workspace, status, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_rope_attention_decode(int kv_dtype, const float *q, const float *k, const float *v, const uint32_t *params,
                               const float *cos_table, const float *sin_table, void *k_cache, void *v_cache, float *out,
                               uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint64_t ld, uint32_t max_seq, float scale,
                               void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
  if (kv_dtype != CUTB_F32 && kv_dtype != CUTB_F16) {
    set_last_error("rope_attention: cache dtype must be fp32 or fp16");
    return CUTB_ERR_INVALID;
  }
  if (!q || !k || !v || !params || !cos_table || !sin_table || !k_cache || !v_cache || !out || !workspace) {
    set_last_error("rope_attention: null pointer");
    return CUTB_ERR_INVALID;
  }
  if (n_heads == 0 || n_kv_heads == 0 || n_heads % n_kv_heads || n_heads / n_kv_heads > 8 || head_dim == 0 || head_dim > 128 ||
      head_dim % 2 || ld < (uint64_t)n_kv_heads * head_dim || max_seq == 0) {
    set_last_error("rope_attention: need n_heads = n_kv_heads * (1..8), even head_dim <= 128, ld >= n_kv_heads * head_dim, max_seq > 0");
    return CUTB_ERR_INVALID;
  }
  if (reinterpret_cast<uintptr_t>(workspace) % 16 || workspace_bytes < attention_workspace_bytes(n_heads, n_kv_heads, head_dim, max_seq)) {
    set_last_error("rope_attention: workspace must be 16-byte aligned and hold %llu bytes",
                   (unsigned long long)attention_workspace_bytes(n_heads, n_kv_heads, head_dim, max_seq));
    return CUTB_ERR_INVALID;
  }
  return rope_attention_decode_launch(kv_dtype, q, k, v, params, cos_table, sin_table, k_cache, v_cache, out, n_heads, n_kv_heads,
                                      head_dim, ld, max_seq, scale, workspace, status, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_dequant(int format, const void *raw, uint64_t raw_bytes, float *out, uint32_t rows, uint32_t cols, uint32_t ldo,
                 void *stream) {
  if (format < CUTB_Q8_0 || format > CUTB_Q5_0) {
    set_last_error("dequant: unknown format %d", format);
    return CUTB_ERR_INVALID;
  }
  if (rows == 0 || cols == 0) return CUTB_OK;
  if (!raw || !out) {
    set_last_error("dequant: null pointer");
    return CUTB_ERR_INVALID;
  }
  if (cols % block_elems(format) != 0) {
    set_last_error("dequant: cols=%u is not a multiple of the block size %u", cols, block_elems(format));
    return CUTB_ERR_INVALID;
  }
  if (ldo < cols) {
    set_last_error("dequant: ldo (%u) < cols (%u)", ldo, cols);
    return CUTB_ERR_INVALID;
  }
  const uint64_t need = (uint64_t)rows * row_bytes(format, cols);
  if (raw_bytes < need) {
    set_last_error("dequant: raw holds %llu bytes, shape needs %llu", (unsigned long long)raw_bytes, (unsigned long long)need);
    return CUTB_ERR_INVALID;
  }
  return dequant_launch(format, raw, out, rows, cols, ldo, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_transpose_q4(const void *in, void *out, uint32_t N, uint32_t K, uint32_t stride_in, uint32_t stride_out,
                      void *stream) {
  // same argument checks as TransposeQ4NibbleOpNode (TransposeQ4NibbleOp.cpp:15-20)
  if (N % 2 != 0) {
    set_last_error("TransposeQ4: N must be even");
    return CUTB_ERR_INVALID;
  }
  if (K % 32 != 0) {
    set_last_error("TransposeQ4: K must be a multiple of 32");
    return CUTB_ERR_INVALID;
  }
  if (N == 0 || K == 0) return CUTB_OK;
  if (!in || !out) {
    set_last_error("TransposeQ4: null pointer");
    return CUTB_ERR_INVALID;
  }
  if (stride_in < K / 2 || stride_out < N / 2) {
    set_last_error("TransposeQ4: strides (%u, %u) too small for N=%u K=%u", stride_in, stride_out, N, K);
    return CUTB_ERR_INVALID;
  }
  return transpose_q4_launch(in, out, N, K, stride_in, stride_out, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_batched_kv_write(int kv_dtype, const float *k_in, const float *v_in, uint32_t k_stride, uint32_t v_stride,
                          const uint32_t *positions, const float *cos_table, const float *sin_table, void *k_cache, void *v_cache,
                          uint32_t n_tokens, uint32_t kv_dim, uint32_t head_dim, uint64_t ld, uint32_t max_seq, int *status, void *stream) {
  if ((kv_dtype != CUTB_F32 && kv_dtype != CUTB_F16) || !k_in || !v_in || !positions || !cos_table || !sin_table || !k_cache || !v_cache) {
    set_last_error("batched_kv_write: null pointer or cache dtype not fp32 / fp16");
    return CUTB_ERR_INVALID;
  }
  if (head_dim == 0 || head_dim % 2 || kv_dim % head_dim || ld < kv_dim || k_stride < kv_dim || v_stride < kv_dim || max_seq == 0) {
    set_last_error("batched_kv_write: head_dim must be even and divide kv_dim; ld, k_stride, v_stride >= kv_dim; max_seq > 0");
    return CUTB_ERR_INVALID;
  }
  return batched_kv_write_launch(kv_dtype, k_in, v_in, k_stride, v_stride, positions, cos_table, sin_table, k_cache, v_cache, n_tokens,
                                 kv_dim, head_dim, ld, max_seq, status, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_batched_attention(int kv_dtype, const float *q_in, uint32_t q_stride, const void *k_cache, const void *v_cache,
                           const uint32_t *positions, const float *cos_table, const float *sin_table, float *out, uint32_t out_stride,
                           uint32_t n_tokens, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint64_t ld, uint32_t max_seq,
                           float scale, int *status, void *stream) {
  if ((kv_dtype != CUTB_F32 && kv_dtype != CUTB_F16) || !q_in || !k_cache || !v_cache || !positions || !cos_table || !sin_table || !out) {
    set_last_error("batched_attention: null pointer or cache dtype not fp32 / fp16");
    return CUTB_ERR_INVALID;
  }
  if (n_heads == 0 || n_kv_heads == 0 || n_heads % n_kv_heads || n_heads / n_kv_heads > 8 || head_dim == 0 || head_dim > 128 ||
      head_dim % 2 || ld < (uint64_t)n_kv_heads * head_dim || q_stride < n_heads * head_dim || out_stride < n_heads * head_dim ||
      max_seq == 0) {
    set_last_error("batched_attention: need n_heads = n_kv_heads * (1..8), even head_dim <= 128, strides >= n_heads * head_dim");
    return CUTB_ERR_INVALID;
  }
  return batched_attention_launch(kv_dtype, q_in, q_stride, k_cache, v_cache, positions, cos_table, sin_table, out, out_stride, n_tokens,
                                  n_heads, n_kv_heads, head_dim, ld, max_seq, scale, status, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_copy_batch(const cutb_copy_range *table, uint32_t n, uint64_t max_bytes, void *stream) {
  if (n == 0) return CUTB_OK;
  if (!table || n > 65535) {
    set_last_error("copy_batch: null table or more than 65535 ranges");
    return CUTB_ERR_INVALID;
  }
  // (the ranges themselves are read on the device: their alignment is the caller's contract)
  uint64_t blocks = (max_bytes / 16 + 2047) / 2048;  // about eight vectors per thread
  if (blocks < 1) blocks = 1;
  if (blocks > 64) blocks = 64;
  return copy_batch_launch(table, n, (uint32_t)blocks, reinterpret_cast<cudaStream_t>(stream));
}

int cutb_glu_pairs(const float *in, float *out, uint32_t rows, uint32_t cols_out, uint64_t ldi, uint64_t ldo, int unary_op, void *stream) {
  if (rows == 0 || cols_out == 0) return CUTB_OK;
  if (!in || !out || ldi % 2 || ldi < 2ull * cols_out || ldo < cols_out || reinterpret_cast<uintptr_t>(in) % 8) {
    set_last_error("glu_pairs: null pointer, odd or short ldi, short ldo, or input not 8-byte aligned");
    return CUTB_ERR_INVALID;
  }
  return glu_pairs_launch(in, out, rows, cols_out, ldi, ldo, unary_op, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
