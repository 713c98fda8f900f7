"""ctypes bindings of the CPU checker (oracle/cut_oracle.c) and, when present,
of the reference's own GGUF reader (oracle/_ref/libcutref.so).

TEST INFRASTRUCTURE ONLY: imported by tests, the smoke check and the benchmark's
CPU-baseline leg; never by the product package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libcutref.so")
_REF_RUNNER_PATH = os.path.join(_HERE, "_ref", "libcutref_runner.so")

Q8_0, Q4_0, Q4_K, Q5_K, Q6_K, BF16, Q4_1, Q5_0 = 0, 1, 2, 3, 4, 5, 6, 7  # from Q5_K on: dequant operator only
BLOCK_ELEMS = {Q8_0: 32, Q4_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256, BF16: 1, Q4_1: 32, Q5_0: 32}
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18, Q4_K: 144, Q5_K: 176, Q6_K: 210, BF16: 2, Q4_1: 20, Q5_0: 22}


def build(force: bool = False) -> None:
    """Compile the checker (and the reference helper when its sources exist)."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "cut_oracle.c"))
    ):
        subprocess.run(["make", "-C", _HERE, "_build/liboracle.so"], check=True, capture_output=True)
    # the reference helpers are rebuilt only where a checkout of the reference is named (REF_ROOT in the
    # environment, else the place this build keeps it); elsewhere the prebuilt files are used as they are
    sibling = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")  # a checkout next to this repository
    ref_root = os.environ.get("REF_ROOT") or (sibling if os.path.isdir(os.path.join(sibling, "interface", "loader", "gguf")) else "")
    subprocess.run(["make", "-C", _HERE, "ref", f"REF_ROOT={ref_root}"], check=True, capture_output=True)
    # the reference's own CUDA matmul kernels as cubins (NVRTC, as its backend compiles them; no GPU needed)
    if ref_root:
        try:
            from . import build_ref_cuda
        except ImportError:
            import build_ref_cuda  # the module run from its own folder
        cuda_dir = os.path.join(_HERE, "_ref", "cuda")
        if force or not all(os.path.exists(os.path.join(cuda_dir, k + ".cubin")) for k in build_ref_cuda.KERNELS):
            try:
                build_ref_cuda.build(ref_root, cuda_dir)
            except Exception as e:  # noqa: BLE001  (no NVRTC bindings here: the GPU-side checker is simply absent)
                print(f"oracle: reference CUDA kernels not built: {e}")


_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16_runner.restype = C.c_uint16
        _lib.orc_f32_to_f16_runner.argtypes = [C.c_float]
        _lib.orc_f32_to_f16_trunc.restype = C.c_uint16
        _lib.orc_f32_to_f16_trunc.argtypes = [C.c_float]
        _lib.orc_epilogue.restype = C.c_float
        _lib.orc_epilogue.argtypes = [C.c_float, C.c_int, C.c_int, C.c_float]
        _lib.orc_requant_q4k_affine.restype = C.c_int
        _lib.orc_f32_to_f16_rne.restype = C.c_uint16
        _lib.orc_f32_to_f16_rne.argtypes = [C.c_float]
        _lib.orc_argreduce.restype = C.c_float
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF_PATH)


def have_ref_runner() -> bool:
    return os.path.exists(_REF_RUNNER_PATH)


_ref_runner = None


def ref_runner() -> C.CDLL:
    """The reference runner's own re-encoders (interface/runner/llama/llama.cpp:445-619), compiled from
    its unmodified source: what the restatements in cut_oracle.c are pinned against."""
    global _ref_runner
    if _ref_runner is None:
        _ref_runner = C.CDLL(_REF_RUNNER_PATH)
        _ref_runner.cutref_runner_f32_to_f16.restype = C.c_uint16
        _ref_runner.cutref_runner_f32_to_f16.argtypes = [C.c_float]
        _ref_runner.cutref_runner_f16_to_f32.restype = C.c_float
        _ref_runner.cutref_runner_f16_to_f32.argtypes = [C.c_uint16]
        _ref_runner.cutref_runner_requant_q4k_affine.restype = C.c_int
    return _ref_runner


def ref_runner_quantize_rows_q8_0(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    values = np.empty(x.size, dtype=np.int8)
    scales = np.empty(x.size // 32, dtype=np.uint16)
    ref_runner().cutref_runner_quantize_rows_q8_0(_p(x), C.c_size_t(x.size), _p(values), _p(scales))
    return values, scales


def ref_runner_requant_q4k_affine(raw, N: int, K: int):
    raw = _u8(raw)
    packedT = np.empty((K, N // 2), dtype=np.uint8)
    scalesT = np.empty((2 * (K // 32), N), dtype=np.uint16)
    ps, ss = C.c_size_t(0), C.c_size_t(0)
    rc = ref_runner().cutref_runner_requant_q4k_affine(_p(raw), C.c_size_t(raw.size), C.c_uint32(N), C.c_uint32(K), _p(packedT),
                                                       C.c_size_t(packedT.size), _p(scalesT), C.c_size_t(scalesT.size),
                                                       C.byref(ps), C.byref(ss))
    if rc != 1:
        raise ValueError(f"the reference declined the shape or the buffers were too small (rc {rc})")
    assert ps.value == packedT.size and ss.value == scalesT.size
    return packedT, scalesT


def ref() -> C.CDLL:
    global _ref
    if _ref is None:
        _ref = C.CDLL(_REF_PATH)
        _ref.cutref_last_error.restype = C.c_char_p
        _ref.cutref_tensor_elements.restype = C.c_long
    return _ref


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.uint8).reshape(-1)


def row_bytes(fmt: int, K: int) -> int:
    be = BLOCK_ELEMS[fmt]
    return (K + be - 1) // be * BLOCK_BYTES[fmt]


# ---------------------------------------------------------------- fp16 helpers
def f16_to_f32(bits) -> np.ndarray:
    b = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(b.shape, dtype=np.float32)
    lib().orc_f16_to_f32_array(_p(b), _p(out), C.c_size_t(b.size))
    return out


def f32_to_f16_runner(x: float) -> int:
    return int(lib().orc_f32_to_f16_runner(C.c_float(x)))


def f32_to_f16_trunc(x: float) -> int:
    return int(lib().orc_f32_to_f16_trunc(C.c_float(x)))


# ------------------------------------------------------------------- dequant
def dequant(fmt: int, raw, n_elements: int) -> np.ndarray:
    raw = _u8(raw)
    out = np.empty(n_elements, dtype=np.float32)
    lib().orc_dequant(C.c_int(fmt), _p(raw), _p(out), C.c_size_t(n_elements))
    return out


def dequant_rows(fmt: int, raw, rows: int, cols: int, ldo: int | None = None) -> np.ndarray:
    raw = _u8(raw)
    ldo = cols if ldo is None else ldo
    out = np.zeros((rows, ldo), dtype=np.float32)
    lib().orc_dequant_rows(C.c_int(fmt), _p(raw), _p(out), C.c_size_t(rows), C.c_size_t(cols), C.c_size_t(ldo))
    return out


# -------------------------------------------------- loader / runner re-encodes
def q8_separate(raw, rows: int, cols: int):
    raw = _u8(raw)
    values = np.empty((rows, cols), dtype=np.int8)
    scales = np.empty((rows, cols // 32), dtype=np.uint16)
    lib().orc_q8_separate(_p(raw), C.c_size_t(rows), C.c_size_t(cols), _p(values), _p(scales))
    return values, scales


def q4_separate(raw, rows: int, cols: int):
    raw = _u8(raw)
    packed = np.empty((rows, cols // 2), dtype=np.uint8)
    scales = np.empty((rows, cols // 32), dtype=np.uint16)
    lib().orc_q4_separate(_p(raw), C.c_size_t(rows), C.c_size_t(cols), _p(packed), _p(scales))
    return packed, scales


def transpose_q4(packed: np.ndarray, N: int, K: int, stride_in: int | None = None, stride_out: int | None = None):
    """[N, stride_in] GGML-packed nibbles -> [K, stride_out] (low nibble = even n)."""
    stride_in = K // 2 if stride_in is None else stride_in
    stride_out = N // 2 if stride_out is None else stride_out
    src = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.zeros((K, stride_out), dtype=np.uint8)
    lib().orc_transpose_q4(_p(src), _p(out), C.c_size_t(N), C.c_size_t(K), C.c_size_t(stride_in), C.c_size_t(stride_out))
    return out


def requant_q4k_affine(raw, N: int, K: int):
    raw = _u8(raw)
    packedT = np.empty((K, N // 2), dtype=np.uint8)
    scalesT = np.empty((2 * (K // 32), N), dtype=np.uint16)
    ok = lib().orc_requant_q4k_affine(_p(raw), C.c_size_t(raw.size), C.c_uint32(N), C.c_uint32(K), _p(packedT), _p(scalesT))
    if not ok:
        raise ValueError("shape not re-encodable (K % 256 or N % 2)")
    return packedT, scalesT


def quantize_rows_q8_0(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    values = np.empty(x.size, dtype=np.int8)
    scales = np.empty(x.size // 32, dtype=np.uint16)
    lib().orc_quantize_rows_q8_0(_p(x), C.c_size_t(x.size), _p(values), _p(scales))
    return values, scales


def epilogue(v: float, fusion_type: int, op: int, d: float = 0.0) -> float:
    return float(lib().orc_epilogue(C.c_float(v), C.c_int(fusion_type), C.c_int(op), C.c_float(d)))


# -------------------------------------------------------------------- matmul
def qmatmul_planes(q4: bool, affine: bool, A, B, S, M: int, K: int, N: int, *, lda=None, ldb=None, lds=None,
                   D=None, fusion_type=0, fusion_op=0, acc64=False) -> np.ndarray:
    """C[M,N] = A[M,K] * W, W in the reference's [K,N] plane layout (strides in elements)."""
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = _u8(B)
    S = np.ascontiguousarray(S, dtype=np.uint16)
    lda = K if lda is None else lda
    ldb = (N // 2 if q4 else N) if ldb is None else ldb
    lds = N if lds is None else lds
    Cm = np.zeros((M, N), dtype=np.float32)
    Dp = None if D is None else np.ascontiguousarray(D, dtype=np.float32)
    lib().orc_qmatmul_planes(C.c_int(int(q4)), C.c_int(int(affine)), _p(A), _p(B), _p(S), _p(Cm),
                             _p(Dp) if Dp is not None else None, C.c_size_t(M), C.c_size_t(K), C.c_size_t(N),
                             C.c_size_t(lda), C.c_size_t(ldb), C.c_size_t(lds), C.c_size_t(N), C.c_size_t(N),
                             C.c_int(fusion_type), C.c_int(fusion_op), C.c_int(int(acc64)))
    return Cm


def qmatmul_blocks(fmt: int, A, W, M: int, K: int, N: int, *, D=None, fusion_type=0, fusion_op=0,
                   acc64=True) -> np.ndarray:
    """C[M,N] = A[M,K] * dequant(W)^T, W = N rows of GGUF blocks."""
    A = np.ascontiguousarray(A, dtype=np.float32).reshape(M, K)
    W = _u8(W)
    Cm = np.zeros((M, N), dtype=np.float32)
    Dp = None if D is None else np.ascontiguousarray(D, dtype=np.float32)
    lib().orc_qmatmul_blocks(C.c_int(fmt), _p(A), _p(W), _p(Cm), _p(Dp) if Dp is not None else None,
                             C.c_size_t(M), C.c_size_t(K), C.c_size_t(N), C.c_size_t(K), C.c_size_t(N),
                             C.c_size_t(N), C.c_int(fusion_type), C.c_int(fusion_op), C.c_int(int(acc64)))
    return Cm


def qmatmul_blocks_fast(fmt: int, A, W, M: int, K: int, N: int) -> np.ndarray:
    A = np.ascontiguousarray(A, dtype=np.float32).reshape(M, K)
    W = _u8(W)
    Cm = np.zeros((M, N), dtype=np.float32)
    lib().orc_qmatmul_blocks_fast(C.c_int(fmt), _p(A), _p(W), _p(Cm), C.c_size_t(M), C.c_size_t(K), C.c_size_t(N),
                                  C.c_size_t(K), C.c_size_t(N))
    return Cm


def matmul_dense(A, Wf, *, acc64=False) -> np.ndarray:
    """C[M,N] = A[M,K] * Wf[N,K]^T with the reference tests' scalar loop."""
    A = np.ascontiguousarray(A, dtype=np.float32)
    Wf = np.ascontiguousarray(Wf, dtype=np.float32)
    M, K = A.shape
    N = Wf.shape[0]
    Cm = np.zeros((M, N), dtype=np.float32)
    lib().orc_matmul_dense(_p(A), _p(Wf), _p(Cm), C.c_size_t(M), C.c_size_t(K), C.c_size_t(N), C.c_size_t(K),
                           C.c_size_t(K), C.c_size_t(N), C.c_int(int(acc64)))
    return Cm


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


# ------------------------------------------ the reference's own reader (_ref)
_TYPE_NAME = {Q8_0: "Q8_0", Q4_0: "Q4_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", BF16: "BF16", Q4_1: "Q4_1", Q5_0: "Q5_0"}


def _with_gguf(fmt: int, raw, rows: int, cols: int, fn):
    from .gguf_file import write_gguf

    d = "/dev/shm" if os.path.isdir("/dev/shm") else None
    fd, path = tempfile.mkstemp(suffix=".gguf", dir=d)
    os.close(fd)
    try:
        write_gguf(path, [("w", _TYPE_NAME[fmt], (rows, cols), _u8(raw))])
        return fn(path.encode())
    finally:
        os.unlink(path)


def ref_write_file(fmt: int, raw, rows: int, cols: int) -> str:
    """Writes a one-tensor GGUF file for the reference's reader; caller unlinks it."""
    from .gguf_file import write_gguf

    d = "/dev/shm" if os.path.isdir("/dev/shm") else None
    fd, path = tempfile.mkstemp(suffix=".gguf", dir=d)
    os.close(fd)
    write_gguf(path, [("w", _TYPE_NAME[fmt], (rows, cols), _u8(raw))])
    return path


def ref_dequant_path(path: str, rows: int, cols: int) -> np.ndarray:
    """GGUFReader(path).read_tensor_f32("w"): the reference's file read + CPU dequantiser."""
    out = np.empty(rows * cols, dtype=np.float32)
    rc = ref().cutref_read_f32(path.encode(), b"w", _p(out), C.c_size_t(out.size))
    if rc:
        raise RuntimeError(ref().cutref_last_error().decode())
    return out.reshape(rows, cols)


def ref_dequant(fmt: int, raw, rows: int, cols: int) -> np.ndarray:
    """Dequantise through the reference's GGUFReader::read_tensor_f32."""
    def run(path):
        out = np.empty(rows * cols, dtype=np.float32)
        rc = ref().cutref_read_f32(path, b"w", _p(out), C.c_size_t(out.size))
        if rc:
            raise RuntimeError(ref().cutref_last_error().decode())
        return out.reshape(rows, cols)

    return _with_gguf(fmt, raw, rows, cols, run)


def ref_separate(fmt: int, raw, rows: int, cols: int):
    """Plane separation through the reference's read_tensor_q8/q4_separated."""
    def run(path):
        r, c = C.c_uint32(), C.c_uint32()
        scales = np.empty((rows, cols // 32), dtype=np.uint16)
        if fmt == Q8_0:
            vals = np.empty((rows, cols), dtype=np.int8)
            rc = ref().cutref_read_q8_separated(path, b"w", _p(vals), _p(scales), C.byref(r), C.byref(c))
        else:
            vals = np.empty((rows, cols // 2), dtype=np.uint8)
            rc = ref().cutref_read_q4_separated(path, b"w", _p(vals), _p(scales), C.byref(r), C.byref(c))
        if rc:
            raise RuntimeError(ref().cutref_last_error().decode())
        assert (r.value, c.value) == (rows, cols)
        return vals, scales

    return _with_gguf(fmt, raw, rows, cols, run)


# ------------------------------------------------------ layer ops next to the matmul
def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, dim = (1, x.shape[0]) if x.ndim == 1 else x.shape
    w = np.ascontiguousarray(weight, dtype=np.float32)
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), _p(y), C.c_size_t(rows), C.c_size_t(dim), C.c_size_t(dim), C.c_float(eps))
    return y


def embedding(indices: np.ndarray, table: np.ndarray) -> np.ndarray:
    """table [vocab, pad4(dim)] float32 -> [n, pad4(dim)]."""
    idx = np.ascontiguousarray(indices, dtype=np.uint32)
    t = np.ascontiguousarray(table, dtype=np.float32)
    out = np.empty((idx.size, t.shape[1]), dtype=np.float32)
    lib().orc_embedding(_p(idx), _p(t), _p(out), C.c_size_t(idx.size), C.c_size_t(t.shape[1]))
    return out


def embedding_col(indices: np.ndarray, matrix: np.ndarray, scales: np.ndarray | None = None) -> np.ndarray:
    """matrix [dim, vocab_stride] as float16 bits (uint16) or int8 (+ scales [dim / 32, scale_stride] float16 bits)."""
    idx = np.ascontiguousarray(indices, dtype=np.uint32)
    dim, vstride = matrix.shape
    fmt = 1 if matrix.dtype == np.int8 else 0
    m = np.ascontiguousarray(matrix)
    sc = np.ascontiguousarray(scales, dtype=np.uint16) if scales is not None else np.zeros((1, 1), dtype=np.uint16)
    ld = (dim + 3) // 4 * 4
    out = np.zeros((idx.size, ld), dtype=np.float32)
    lib().orc_embedding_col(C.c_int(fmt), _p(idx), _p(m), _p(sc), _p(out), C.c_size_t(idx.size), C.c_size_t(dim), C.c_size_t(vstride),
                            C.c_size_t(sc.shape[1]), C.c_size_t(ld))
    return out


def argreduce(v: np.ndarray, is_max: bool = True) -> float:
    v = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
    return float(lib().orc_argreduce(_p(v), C.c_size_t(v.size), C.c_int(1 if is_max else 0)))


def f32_to_f16_rne(x: float) -> int:
    return int(lib().orc_f32_to_f16_rne(C.c_float(x)))


def rope_kv_write(q, k, v, pos: int, cos_t, sin_t, k_cache: np.ndarray, v_cache: np.ndarray, head_dim: int) -> np.ndarray:
    """Writes row `pos` of the caches ([max_seq, ld], float32 or float16) in place; returns roped q."""
    q, k, v = (np.ascontiguousarray(a, dtype=np.float32) for a in (q, k, v))
    cos_t, sin_t = (np.ascontiguousarray(a, dtype=np.float32) for a in (cos_t, sin_t))
    assert k_cache.dtype == v_cache.dtype and k_cache.dtype in (np.float32, np.float16)
    assert k_cache.flags.c_contiguous and v_cache.flags.c_contiguous
    out = np.empty_like(q)
    lib().orc_rope_kv_write(C.c_int(int(k_cache.dtype == np.float16)), _p(q), _p(k), _p(v), C.c_uint32(pos), _p(cos_t), _p(sin_t),
                            _p(k_cache), _p(v_cache), _p(out), C.c_size_t(q.size), C.c_size_t(k.size), C.c_size_t(head_dim),
                            C.c_size_t(k_cache.shape[1]))
    return out


def attention(q, k_cache: np.ndarray, v_cache: np.ndarray, seq_len: int, n_heads: int, n_kv_heads: int, head_dim: int,
              scale: float | None = None) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    assert k_cache.dtype == v_cache.dtype and k_cache.dtype in (np.float32, np.float16)
    k_cache, v_cache = np.ascontiguousarray(k_cache), np.ascontiguousarray(v_cache)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    if scale is None:
        scale = 1.0 / float(np.sqrt(np.float32(head_dim)))
    lib().orc_attention(C.c_int(int(k_cache.dtype == np.float16)), _p(q), _p(k_cache), _p(v_cache), C.c_size_t(seq_len), _p(out),
                        C.c_size_t(n_heads), C.c_size_t(n_kv_heads), C.c_size_t(head_dim), C.c_size_t(k_cache.shape[1]),
                        C.c_float(scale))
    return out

