"""ctypes view of libcutb.so, laid out exactly as include/cutb.h declares it.

There is no fallback: if the library has not been built, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcutb.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_TIMEOUT, ERR_RANGE = range(7)
Q8_0, Q4_0, Q4_K, Q5_K, Q6_K, BF16, Q4_1, Q5_0 = 0, 1, 2, 3, 4, 5, 6, 7  # from Q5_K on: cutb_dequant only
F32, F16 = 0, 1
LAYOUT_GGUF_BLOCKS, LAYOUT_KN_PLANES = 0, 1
FUSION_NONE, FUSION_UNARY, FUSION_BINARY = 0, 1, 2
VARIANT_AUTO, VARIANT_GENERIC, VARIANT_GEMV_MMA, VARIANT_GEMM_TC, VARIANT_GEMV_PLANES = -1, 0, 1, 2, 3
FLAG_NO_OVERLAP = 1
FLAG_ACT_16BIT = 2
FLAG_A_RMSNORM = 4
FLAG_GLU_PAIRS = 8
FLAG_STAGE_PER_CTA = 16

# every symbol include/cutb.h declares
EXPORTS = [
    "cutb_qmatmul_workspace_bytes", "cutb_qmatmul_select_variant", "cutb_qmatmul", "cutb_qmatmul_decode_noalloc",
    "cutb_qmatmul_scatter", "cutb_peer_exchange", "cutb_copy_batch",
    "cutb_peer_buffer_alloc", "cutb_peer_buffer_open", "cutb_peer_buffer_close", "cutb_peer_buffer_free",
    "cutb_rmsnorm", "cutb_embedding", "cutb_embedding_col", "cutb_embedding_blocks", "cutb_argreduce",
    "cutb_rope_kv_write", "cutb_attention_workspace_bytes", "cutb_attention_decode", "cutb_rope_attention_decode",
    "cutb_batched_kv_write", "cutb_batched_attention", "cutb_glu_pairs",
    "cutb_dequant", "cutb_separate_blocks", "cutb_transpose_2d", "cutb_requant_q4k_affine", "cutb_quantize_rows_q8_0", "cutb_requant_q8_0_blocks",
    "cutb_transpose_q4", "cutb_version", "cutb_status_string", "cutb_last_error", "cutb_device_sm_count",
    "cutb_variant_name",
]


class QMatmulDesc(C.Structure):
    _fields_ = [
        ("format", C.c_int32), ("layout", C.c_int32), ("affine", C.c_int32), ("a_dtype", C.c_int32),
        ("M", C.c_uint32), ("K", C.c_uint32), ("N", C.c_uint32),
        ("A", C.c_void_p), ("lda", C.c_uint32),
        ("W", C.c_void_p), ("W_bytes", C.c_uint64),
        ("scales", C.c_void_p), ("ldb", C.c_uint32), ("lds", C.c_uint32),
        ("C", C.c_void_p), ("ldc", C.c_uint32),
        ("D", C.c_void_p), ("ldd", C.c_uint32),
        ("fusion_type", C.c_int32), ("fusion_op", C.c_int32), ("variant", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
        ("status", C.c_void_p),
        ("flags", C.c_uint32),
        ("a_norm_weight", C.c_void_p), ("a_norm_eps", C.c_float),
    ]


MAX_PEERS = 8


class PeerScatter(C.Structure):
    _fields_ = [
        ("world", C.c_uint32), ("rank", C.c_uint32), ("ldc_total", C.c_uint32), ("n_offset", C.c_uint32),
        ("C_peers", C.c_void_p * MAX_PEERS), ("flag_peers", C.c_void_p * MAX_PEERS),
    ]


class CutbError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"cutb status {status}: {message}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cut_b200.build` (there is no CPU fallback)")
        l = C.CDLL(LIB_PATH)
        l.cutb_qmatmul_workspace_bytes.restype = C.c_uint64
        l.cutb_qmatmul_workspace_bytes.argtypes = [C.POINTER(QMatmulDesc)]
        l.cutb_qmatmul_select_variant.restype = C.c_int
        l.cutb_qmatmul_select_variant.argtypes = [C.POINTER(QMatmulDesc)]
        l.cutb_qmatmul.restype = C.c_int
        l.cutb_qmatmul.argtypes = [C.POINTER(QMatmulDesc), C.c_void_p]
        l.cutb_qmatmul_decode_noalloc.restype = C.c_int
        l.cutb_qmatmul_decode_noalloc.argtypes = [C.POINTER(QMatmulDesc), C.c_void_p]
        l.cutb_qmatmul_scatter.restype = C.c_int
        l.cutb_qmatmul_scatter.argtypes = [C.POINTER(QMatmulDesc), C.POINTER(PeerScatter), C.c_void_p]
        l.cutb_copy_batch.restype = C.c_int
        l.cutb_copy_batch.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p]
        l.cutb_peer_exchange.restype = C.c_int
        l.cutb_peer_exchange.argtypes = [C.POINTER(PeerScatter), C.c_void_p, C.c_void_p, C.c_void_p]
        l.cutb_peer_buffer_alloc.restype = C.c_int
        l.cutb_peer_buffer_alloc.argtypes = [C.c_uint64, C.POINTER(C.c_void_p), C.c_char_p]
        l.cutb_peer_buffer_open.restype = C.c_int
        l.cutb_peer_buffer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        l.cutb_peer_buffer_close.restype = C.c_int
        l.cutb_peer_buffer_close.argtypes = [C.c_void_p]
        l.cutb_peer_buffer_free.restype = C.c_int
        l.cutb_peer_buffer_free.argtypes = [C.c_void_p]
        l.cutb_dequant.restype = C.c_int
        l.cutb_dequant.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                   C.c_void_p]
        l.cutb_rmsnorm.restype = C.c_int
        l.cutb_rmsnorm.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_float, C.c_void_p]
        l.cutb_embedding.restype = C.c_int
        l.cutb_embedding.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
        l.cutb_embedding_col.restype = C.c_int
        l.cutb_embedding_col.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                         C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
        l.cutb_embedding_blocks.restype = C.c_int
        l.cutb_embedding_blocks.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                            C.c_void_p, C.c_void_p]
        l.cutb_requant_q8_0_blocks.restype = C.c_int
        l.cutb_requant_q8_0_blocks.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p]
        l.cutb_argreduce.restype = C.c_int
        l.cutb_argreduce.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]
        l.cutb_rope_kv_write.restype = C.c_int
        l.cutb_rope_kv_write.argtypes = [C.c_int] + [C.c_void_p] * 9 + [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint32,
                                                                        C.c_void_p, C.c_void_p]
        l.cutb_attention_workspace_bytes.restype = C.c_uint64
        l.cutb_attention_workspace_bytes.argtypes = [C.c_uint32] * 4
        l.cutb_attention_decode.restype = C.c_int
        l.cutb_attention_decode.argtypes = [C.c_int] + [C.c_void_p] * 5 + [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint32,
                                                                           C.c_float, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
        l.cutb_rope_attention_decode.restype = C.c_int
        l.cutb_rope_attention_decode.argtypes = [C.c_int] + [C.c_void_p] * 9 + [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint32,
                                                                                C.c_float, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
        l.cutb_batched_kv_write.restype = C.c_int
        l.cutb_batched_kv_write.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32] + [C.c_void_p] * 5 + [
            C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint32, C.c_void_p, C.c_void_p]
        l.cutb_batched_attention.restype = C.c_int
        l.cutb_batched_attention.argtypes = [C.c_int, C.c_void_p, C.c_uint32] + [C.c_void_p] * 6 + [
            C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint32, C.c_float, C.c_void_p, C.c_void_p]
        l.cutb_glu_pairs.restype = C.c_int
        l.cutb_glu_pairs.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint64, C.c_int, C.c_void_p]
        l.cutb_separate_blocks.restype = C.c_int
        l.cutb_separate_blocks.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p]
        l.cutb_transpose_2d.restype = C.c_int
        l.cutb_transpose_2d.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint64, C.c_void_p]
        l.cutb_requant_q4k_affine.restype = C.c_int
        l.cutb_requant_q4k_affine.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64,
                                              C.c_uint64, C.c_void_p]
        l.cutb_quantize_rows_q8_0.restype = C.c_int
        l.cutb_quantize_rows_q8_0.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
        l.cutb_transpose_q4.restype = C.c_int
        l.cutb_transpose_q4.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                        C.c_void_p]
        l.cutb_version.restype = C.c_int
        l.cutb_status_string.restype = C.c_char_p
        l.cutb_status_string.argtypes = [C.c_int]
        l.cutb_last_error.restype = C.c_char_p
        l.cutb_device_sm_count.restype = C.c_int
        l.cutb_variant_name.restype = C.c_char_p
        l.cutb_variant_name.argtypes = [C.c_int]
        _lib = l
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise CutbError(status, lib().cutb_last_error().decode() or lib().cutb_status_string(status).decode())
