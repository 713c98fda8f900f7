// Internal launchers behind the C ABI (one per kernel family).
#pragma once

#include <cuda_runtime.h>

#include "../../include/cutb.h"

namespace cutb {

// Argument checks shared by the cutb_qmatmul entry points (CUTB_OK or an error code + message).
int check_qmatmul_desc(const cutb_qmatmul_desc *d);

// Decode mat-vec over GGUF blocks (bulk-copy ring + warp MMA).
bool qgemv_blocks_supported(const cutb_qmatmul_desc &d);
// up to four row groups of the mat-vec (a forced variant only; CUTB_VARIANT_AUTO stays within one group)
bool qgemv_blocks_supported_in_groups(const cutb_qmatmul_desc &d);
uint64_t qgemv_blocks_workspace(const cutb_qmatmul_desc &d);
// `scatter` (optional): store the output slice into every rank's full output instead of d.C.
int qgemv_blocks_launch(const cutb_qmatmul_desc &d, cudaStream_t stream, const cutb_peer_scatter *scatter = nullptr);
// Publishes this rank's peer stores of the step and waits (bounded) for every rank's.
int peer_exchange_launch(const cutb_peer_scatter &peers, uint64_t *step_counter, int *status, cudaStream_t stream);

// Any-shape SIMT matmul over GGUF blocks or the reference's [K,N] planes.
int qmatmul_generic_launch(const cutb_qmatmul_desc &d, cudaStream_t stream);

// Decode mat-vec over the reference's [K,N] planes (qgemv_planes.cu).
bool qgemv_planes_supported(const cutb_qmatmul_desc &d);
uint64_t qgemv_planes_workspace(const cutb_qmatmul_desc &d);
int qgemv_planes_launch(const cutb_qmatmul_desc &d, cudaStream_t stream);

// Prefill GEMM over GGUF blocks on tcgen05 tensor cores.
bool qgemm_tc_supported(const cutb_qmatmul_desc &d);
uint64_t qgemm_tc_workspace(const cutb_qmatmul_desc &d);
int qgemm_tc_launch(const cutb_qmatmul_desc &d, cudaStream_t stream);
// the same GEMM for up to 128 activation rows (operand roles swapped, K stages dealt over all SMs); reached through qgemm_tc_*
bool qgemm_skinny_applies(const cutb_qmatmul_desc &d);
uint64_t qgemm_skinny_workspace(const cutb_qmatmul_desc &d);
int qgemm_skinny_launch(const cutb_qmatmul_desc &d, cudaStream_t stream);

int dequant_launch(int format, const void *raw, float *out, uint32_t rows, uint32_t cols, uint32_t ldo,
                   cudaStream_t stream);
// Layer operators next to the matmul (layer_ops.cu).
int rmsnorm_launch(int dtype, const void *x, const void *weight, void *y, uint32_t rows, uint32_t dim, uint64_t ldx, float eps,
                   cudaStream_t stream);
int embedding_launch(const uint32_t *indices, const float *table, float *out, uint64_t n, uint32_t dim, uint32_t vocab, int *status,
                     cudaStream_t stream);
int embedding_col_launch(int format, const uint32_t *indices, const void *matrix, const void *scales, float *out, uint32_t n,
                         uint32_t dim, uint32_t vocab, uint32_t vocab_stride, uint32_t scale_stride, uint32_t out_stride, int *status,
                         cudaStream_t stream);
int requant_q8_0_blocks_launch(int format, const void *raw, void *out, uint64_t rows, uint32_t cols, cudaStream_t stream);
int dequant_gather_launch(int format, const uint32_t *indices, const void *raw, float *out, uint32_t n, uint32_t rows, uint32_t cols,
                          uint32_t ldo, int *status, cudaStream_t stream);
int copy_batch_launch(const cutb_copy_range *table, uint32_t n, uint32_t blocks_per_range, cudaStream_t stream);
int argreduce_launch(int is_max, const float *v, float *out, uint32_t n, cudaStream_t stream);
// Decode-step attention (attention.cu).
int rope_kv_write_launch(int kv_dtype, const float *q, const float *k, const float *v, const uint32_t *params, const float *cosT,
                         const float *sinT, void *kC, void *vC, float *qOut, uint32_t qDim, uint32_t kvDim, uint32_t headDim,
                         uint64_t ld, uint32_t max_seq, int *status, cudaStream_t stream);
int rope_attention_decode_launch(int kv_dtype, const float *q, const float *k, const float *v, const uint32_t *params,
                                 const float *cosT, const float *sinT, void *kC, void *vC, float *out, uint32_t nHeads,
                                 uint32_t nKvHeads, uint32_t headDim, uint64_t ld, uint32_t max_seq, float scale, void *workspace,
                                 int *status, cudaStream_t stream);
int batched_kv_write_launch(int kv_dtype, const float *k_in, const float *v_in, uint32_t k_stride, uint32_t v_stride,
                            const uint32_t *positions, const float *cosT, const float *sinT, void *kC, void *vC, uint32_t n_tokens,
                            uint32_t kvDim, uint32_t headDim, uint64_t ld, uint32_t max_seq, int *status, cudaStream_t stream);
int batched_attention_launch(int kv_dtype, const float *q_in, uint32_t q_stride, const void *kC, const void *vC,
                             const uint32_t *positions, const float *cosT, const float *sinT, float *out, uint32_t out_stride,
                             uint32_t n_tokens, uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint64_t ld, uint32_t max_seq,
                             float scale, int *status, cudaStream_t stream);
// the same on the tensor cores (fp16 cache, head_dim 64 / 128, 16 tokens and more); batched_attention_launch hands over
bool batched_attention_tc_applies(int kv_dtype, const float *q_in, uint32_t q_stride, const void *kC, const void *vC, const float *out,
                                  uint32_t out_stride, uint32_t n_tokens, uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim,
                                  uint64_t ld);
int batched_attention_tc_launch(const float *q_in, uint32_t q_stride, const void *kC, const void *vC, const uint32_t *positions,
                                const float *cosT, const float *sinT, float *out, uint32_t out_stride, uint32_t n_tokens,
                                uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint64_t ld, uint32_t max_seq, float scale,
                                int *status, cudaStream_t stream);
int glu_pairs_launch(const float *in, float *out, uint32_t rows, uint32_t cols_out, uint64_t ldi, uint64_t ldo, int unary_op,
                     cudaStream_t stream);
uint64_t attention_workspace_bytes(uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint32_t max_seq);
int attention_decode_launch(int kv_dtype, const float *q, const void *kC, const void *vC, const uint32_t *params, float *out,
                            uint32_t nHeads, uint32_t nKvHeads, uint32_t headDim, uint64_t ld, uint32_t max_seq, float scale,
                            void *workspace, int *status, cudaStream_t stream);

// Load-time repacks (repack.cu), bit-exact with the reference's CPU loader / runner code.
int separate_launch(int format, const void *raw, void *values, void *scales, uint64_t rows, uint64_t cols, cudaStream_t stream);
int transpose_launch(uint32_t elem_bytes, const void *in, void *out, uint32_t R, uint32_t C, uint64_t ldi, uint64_t ldo,
                     cudaStream_t stream);
int requant_q4k_affine_launch(const void *raw, void *packedT, void *scalesT, uint32_t N, uint32_t K, uint64_t ldp, uint64_t lds,
                              cudaStream_t stream);
int quantize_rows_q8_0_launch(const float *x, void *values, void *scales, uint64_t n, cudaStream_t stream);
int transpose_q4_launch(const void *in, void *out, uint32_t N, uint32_t K, uint32_t stride_in, uint32_t stride_out,
                        cudaStream_t stream);

}  // namespace cutb
