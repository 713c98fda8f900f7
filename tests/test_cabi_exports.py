"""CPU tests of the C-ABI library itself: it loads, exports every symbol the
header declares, and its argument validation answers without a GPU."""
import ctypes as C
import os
import re

import pytest

from cut_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "cutb.h")).read()
    return re.findall(r"CUTB_API\s+[\w\s\*]+?\b(cutb_\w+)\s*\(", text)


def test_library_exports_every_declared_symbol():
    lib = L.lib()
    names = _declared_symbols()
    assert len(names) >= 10
    assert sorted(names) == sorted(L.EXPORTS)
    for n in names:
        assert hasattr(lib, n), n
    assert lib.cutb_version() == 100


def test_descriptor_layout_matches_header():
    # field order and types of cutb_qmatmul_desc as declared in include/cutb.h
    text = open(os.path.join(ROOT, "include", "cutb.h")).read()
    body = re.search(r"typedef struct cutb_qmatmul_desc \{(.*?)\} cutb_qmatmul_desc;", text, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        names = [n.strip().lstrip("*") for n in decl.split(",")]
        first = names[0].split()[-1].lstrip("*")
        fields += [first] + names[1:]
    assert fields == [f[0] for f in L.QMatmulDesc._fields_]
    assert C.sizeof(L.QMatmulDesc) == 168
    assert C.sizeof(L.PeerScatter) == 16 + 2 * 8 * L.MAX_PEERS


def test_validation_needs_no_device():
    lib = L.lib()
    d = L.QMatmulDesc()
    assert lib.cutb_qmatmul(C.byref(d), None) == L.ERR_INVALID
    assert b"empty shape" in lib.cutb_last_error()
    assert lib.cutb_qmatmul(None, None) == L.ERR_INVALID
    assert lib.cutb_qmatmul_select_variant(C.byref(d)) < 0
    assert lib.cutb_qmatmul_workspace_bytes(C.byref(d)) == 0
    assert lib.cutb_dequant(9, None, 0, None, 1, 32, 32, None) == L.ERR_INVALID
    assert lib.cutb_dequant(L.Q4_K, None, 0, None, 1, 100, 100, None) == L.ERR_INVALID
    assert lib.cutb_dequant(L.Q4_K, None, 0, None, 0, 0, 0, None) == L.OK  # empty tensor: nothing to do
    assert lib.cutb_transpose_q4(None, None, 3, 32, 16, 2, None) == L.ERR_INVALID
    assert b"N must be even" in lib.cutb_last_error()
    assert lib.cutb_transpose_q4(None, None, 4, 24, 12, 2, None) == L.ERR_INVALID
    assert lib.cutb_transpose_q4(None, None, 0, 0, 0, 0, None) == L.OK
    assert lib.cutb_status_string(L.ERR_TIMEOUT) == b"device-side wait timed out"
    assert lib.cutb_variant_name(L.VARIANT_GEMV_MMA) == b"QGemvBulkMma"


def test_select_variant_and_workspace_plan_without_device():
    """Variant choice and the split-K workspace size are host logic."""
    lib = L.lib()

    def desc(fmt, M, K, N, dtype=L.F16, layout=L.LAYOUT_GGUF_BLOCKS):
        d = L.QMatmulDesc()
        d.format, d.layout, d.a_dtype = fmt, layout, dtype
        d.M, d.K, d.N, d.lda, d.ldc = M, K, N, K, N
        d.A = d.W = d.C = 256  # never dereferenced here
        d.W_bytes = 1 << 40
        d.variant = L.VARIANT_AUTO
        if layout == L.LAYOUT_KN_PLANES:
            d.scales, d.ldb, d.lds = 256, N, N
        return d

    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q4_0, 1, 4096, 11008))) == L.VARIANT_GEMV_MMA
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q4_0, 12, 4096, 11008))) == L.VARIANT_GEMV_MMA
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q4_0, 16, 2048, 2048))) == L.VARIANT_GEMV_MMA
    # 13 to 16 fp16 rows on 16 M weights and more: the tensor-core GEMM for few tokens (paired rows included), unless the
    # fused RMSNorm, which only the mat-vec has, is asked for
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q4_0, 16, 4096, 11008))) == L.VARIANT_GEMM_TC
    flagged = desc(L.Q4_0, 16, 4096, 11008)
    flagged.flags, flagged.fusion_type, flagged.fusion_op = L.FLAG_GLU_PAIRS, L.FUSION_UNARY, 133
    assert lib.cutb_qmatmul_select_variant(C.byref(flagged)) == L.VARIANT_GEMM_TC
    flagged.flags, flagged.a_norm_weight = L.FLAG_A_RMSNORM, 256
    assert lib.cutb_qmatmul_select_variant(C.byref(flagged)) == L.VARIANT_GEMV_MMA
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q8_0, 8, 4096, 11008, L.F32))) == L.VARIANT_GEMV_MMA
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q4_0, 17, 4096, 11008))) != L.VARIANT_GEMV_MMA
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q8_0, 1, 4096, 4096, L.F32))) == L.VARIANT_GEMV_MMA
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q8_0, 9, 4096, 4096, L.F32))) != L.VARIANT_GEMV_MMA
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q4_0, 1, 96, 8))) == L.VARIANT_GENERIC
    # the reference's [K, N] planes: the coalesced mat-vec up to four rows, strides padded to 4; else the any-shape kernel
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q8_0, 1, 64, 4, L.F32, L.LAYOUT_KN_PLANES))) == L.VARIANT_GEMV_PLANES
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q4_0, 4, 4096, 11008, L.F32, L.LAYOUT_KN_PLANES))) == L.VARIANT_GEMV_PLANES
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q8_0, 5, 64, 4, L.F32, L.LAYOUT_KN_PLANES))) == L.VARIANT_GENERIC
    assert lib.cutb_qmatmul_select_variant(C.byref(desc(L.Q8_0, 1, 64, 6, L.F32, L.LAYOUT_KN_PLANES))) == L.VARIANT_GENERIC  # ldb = 6
    assert lib.cutb_qmatmul_workspace_bytes(C.byref(desc(L.Q8_0, 1, 4096, 4096, L.F32, L.LAYOUT_KN_PLANES))) > 0  # K split over blocks
    assert lib.cutb_variant_name(L.VARIANT_GEMV_PLANES) == b"QGemvPlanes"
    assert lib.cutb_qmatmul_workspace_bytes(C.byref(desc(L.Q4_0, 1, 4096, 11008))) == 0
    # few rows, long K: split over K, partial sums staged in the workspace
    d = desc(L.Q4_0, 8, 28672, 1024)
    d.flags = L.FLAG_STAGE_PER_CTA
    ws = lib.cutb_qmatmul_workspace_bytes(C.byref(d))
    assert ws > 0 and ws % (8 * 1024 * 4) == 0
    # the tensor-core GEMM for few tokens: head / tail slots of every CTA of its K split (43 tiles of 256 rows x 16 units
    # of 256 k over 148 SMs -> runs of 5 units, 138 CTAs), [2 x CTAs][tokens rounded to 8][256] floats
    g = desc(L.Q4_0, 32, 4096, 11008)
    g.variant = L.VARIANT_GEMM_TC
    assert lib.cutb_qmatmul_workspace_bytes(C.byref(g)) == 2 * 138 * 32 * 256 * 4
    g = desc(L.Q4_0, 30, 4096, 11008, L.F32)   # fp32 rows: their fp16 copy comes first
    g.variant = L.VARIANT_GEMM_TC
    assert lib.cutb_qmatmul_workspace_bytes(C.byref(g)) == 30 * 4096 * 2 + 2 * 138 * 32 * 256 * 4
    g = desc(L.Q4_0, 32, 256, 38400)           # more tiles than SMs: no split, no slots
    g.variant = L.VARIANT_GEMM_TC
    assert lib.cutb_qmatmul_workspace_bytes(C.byref(g)) == 0
    # three rows and more: the activations are quantised once per call into the workspace as well
    d.flags = 0
    assert lib.cutb_qmatmul_workspace_bytes(C.byref(d)) > ws
    assert lib.cutb_qmatmul_workspace_bytes(C.byref(desc(L.Q4_0, 2, 4096, 11008))) == 0
