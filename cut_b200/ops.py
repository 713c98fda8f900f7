"""Python harness over the C ABI: torch supplies device memory and streams only.

These wrappers mirror the reference's operator entry points for the path
(runtime/Operations.h:65-93 matmul / matmulUnary / matmulBinary, :459
transposeQ4, :467 dequantize): outputs are allocated by the op, shape errors
raise, and nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _pad4(n: int) -> int:
    return (n + 3) & ~3


def make_desc(A: torch.Tensor, W: torch.Tensor, fmt: int, N: int, *, layout=L.LAYOUT_GGUF_BLOCKS, scales=None,
              affine=False, ldb=0, lds=0, C_out: torch.Tensor | None = None, D: torch.Tensor | None = None,
              fusion_type=L.FUSION_NONE, fusion_op=0, variant=L.VARIANT_AUTO, workspace: torch.Tensor | None = None,
              status: torch.Tensor | None = None, flags: int = 0):
    """Builds a cutb_qmatmul_desc over torch CUDA tensors; returns (desc, C, keepalive)."""
    if A.dim() == 1:
        A = A.unsqueeze(0)
    if A.dim() != 2:
        raise RuntimeError("matmul: A must be 1D or 2D")
    if A.dtype not in (torch.float32, torch.float16):
        raise RuntimeError("matmul: A must be float32 or float16")
    if A.stride(1) != 1:
        A = A.contiguous()
    M, K = A.shape
    if C_out is None:  # paired gate / up rows give one output column per pair
        C_out = torch.empty((M, N // 2 if flags & L.FLAG_GLU_PAIRS else N), dtype=torch.float32, device=A.device)
    d = L.QMatmulDesc()
    d.format, d.layout, d.affine = fmt, layout, int(affine)
    d.a_dtype = L.F32 if A.dtype == torch.float32 else L.F16
    d.M, d.K, d.N = M, K, N
    d.A, d.lda = A.data_ptr(), A.stride(0) if M > 1 else max(A.stride(0), K)
    d.W, d.W_bytes = W.data_ptr(), W.numel() * W.element_size()
    d.scales = scales.data_ptr() if scales is not None else None
    d.ldb, d.lds = ldb, lds
    d.C, d.ldc = C_out.data_ptr(), C_out.stride(0)
    d.D, d.ldd = (D.data_ptr(), D.stride(0)) if D is not None else (None, 0)
    d.fusion_type, d.fusion_op, d.variant = fusion_type, fusion_op, variant
    d.workspace, d.workspace_bytes = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) \
        if workspace is not None else (None, 0)
    d.status = status.data_ptr() if status is not None else None
    d.flags = flags
    return d, C_out, (A, W, scales, D, workspace, status)


def workspace_bytes(desc) -> int:
    return int(L.lib().cutb_qmatmul_workspace_bytes(C.byref(desc)))


def select_variant(desc) -> int:
    return int(L.lib().cutb_qmatmul_select_variant(C.byref(desc)))


def qmatmul(A, W, fmt, N, **kw) -> torch.Tensor:
    """C[M,N] = epilogue(A[M,K] * dequant(W)); allocates C and, if needed, the workspace."""
    d, C_out, keep = make_desc(A, W, fmt, N, **kw)
    need = workspace_bytes(d)
    if need and not d.workspace:
        ws = torch.empty(need, dtype=torch.uint8, device=A.device)
        d.workspace, d.workspace_bytes = ws.data_ptr(), need
        keep = keep + (ws,)
    L.check(L.lib().cutb_qmatmul(C.byref(d), _stream_ptr()))
    return C_out


def launch(desc) -> None:
    """Re-launch a prepared descriptor on the current stream (benchmark inner loop)."""
    L.check(L.lib().cutb_qmatmul(C.byref(desc), _stream_ptr()))


def dequantize(raw: torch.Tensor, fmt: int, rows: int, cols: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Raw GGUF bytes -> float32 [rows, cols]; the row stride is padded to 4 as the
    reference's DequantOpNode does (operators/impl/dequant/DequantOp.cpp:15-17)."""
    ldo = _pad4(cols)
    if out is None:
        out = torch.empty((rows, ldo), dtype=torch.float32, device=raw.device)
    L.check(L.lib().cutb_dequant(fmt, raw.data_ptr(), raw.numel() * raw.element_size(), out.data_ptr(), rows, cols,
                                 out.stride(0), _stream_ptr()))
    return out[:, :cols]


def transpose_q4(packed: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """[N, pad4(K/2)] GGML nibbles -> [K, pad4(N/2)] with even n in the low nibble."""
    if packed.dim() != 2:
        raise RuntimeError("TransposeQ4: input must be 2D")
    out = torch.zeros((K, _pad4(N // 2)), dtype=torch.uint8, device=packed.device)
    L.check(L.lib().cutb_transpose_q4(packed.data_ptr(), out.data_ptr(), N, K, packed.stride(0), out.stride(0),
                                      _stream_ptr()))
    return out


# ---- load-time repacks on the device (bit-exact with the reference's CPU loader / runner) ----
def separate_blocks(raw: torch.Tensor, fmt: int, rows: int, cols: int):
    """Q8_0 / Q4_0 blocks -> (values [rows, cols] int8 or packed nibbles [rows, cols / 2] uint8, scales [rows, cols / 32]
    as int16 bit patterns of f16), as the reference's read_tensor_q8/q4_separated return them."""
    vals = torch.empty((rows, cols if fmt == L.Q8_0 else cols // 2), dtype=torch.int8 if fmt == L.Q8_0 else torch.uint8,
                       device=raw.device)
    scales = torch.empty((rows, cols // 32), dtype=torch.int16, device=raw.device)
    L.check(L.lib().cutb_separate_blocks(fmt, raw.data_ptr(), raw.numel() * raw.element_size(), vals.data_ptr(), scales.data_ptr(),
                                         rows, cols, _stream_ptr()))
    return vals, scales


def transpose_2d(x: torch.Tensor, ldo: int | None = None) -> torch.Tensor:
    """[R, C] of 1- or 2-byte elements -> [C, ldo >= R] (padding zero-filled)."""
    R, Cc = x.shape
    ldo = R if ldo is None else ldo
    out = torch.zeros((Cc, ldo), dtype=x.dtype, device=x.device)
    L.check(L.lib().cutb_transpose_2d(x.element_size(), x.data_ptr(), out.data_ptr(), R, Cc, x.stride(0), ldo, _stream_ptr()))
    return out


def requant_q4k_affine(raw: torch.Tensor, N: int, K: int):
    """Q4_K rows -> (nibbles [K, N / 2] uint8, f16 bit patterns [2 K / 32, N] int16): the runner's affine re-encode."""
    packedT = torch.zeros((K, N // 2), dtype=torch.uint8, device=raw.device)
    scalesT = torch.zeros((2 * (K // 32), N), dtype=torch.int16, device=raw.device)
    L.check(L.lib().cutb_requant_q4k_affine(raw.data_ptr(), raw.numel() * raw.element_size(), packedT.data_ptr(), scalesT.data_ptr(),
                                            N, K, N // 2, N, _stream_ptr()))
    return packedT, scalesT


def quantize_rows_q8_0(x: torch.Tensor):
    """float32 values (multiple of 32) -> (int8 values, f16 scale bit patterns), the runner's Q8_0 requantiser."""
    x = x.contiguous().view(-1)
    vals = torch.empty(x.numel(), dtype=torch.int8, device=x.device)
    scales = torch.empty(x.numel() // 32, dtype=torch.int16, device=x.device)
    L.check(L.lib().cutb_quantize_rows_q8_0(x.data_ptr(), vals.data_ptr(), scales.data_ptr(), x.numel(), _stream_ptr()))
    return vals, scales


# ---- layer operators next to the matmul ----
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * weight over the last dimension (fp32 or fp16, 1-D or 2-D)."""
    x2 = x if x.dim() == 2 else x.view(1, -1)
    if x2.stride(1) != 1 or weight.dtype != x.dtype:
        raise RuntimeError("rmsnorm: contiguous rows and a weight of the input's dtype")
    y = torch.empty_like(x2)
    dt = L.F16 if x.dtype == torch.float16 else L.F32
    L.check(L.lib().cutb_rmsnorm(dt, x2.data_ptr(), weight.data_ptr(), y.data_ptr(), x2.shape[0], x2.shape[1], x2.stride(0), eps,
                                 _stream_ptr()))
    return y.view_as(x)


def embedding(indices: torch.Tensor, table: torch.Tensor, dim: int | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """table [vocab, pad4(dim)] float32, indices int32 -> [n, pad4(dim)]."""
    dim = table.shape[1] if dim is None else dim
    out = torch.empty((indices.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    L.check(L.lib().cutb_embedding(indices.data_ptr(), table.data_ptr(), out.data_ptr(), indices.numel(), dim, table.shape[0],
                                   status.data_ptr() if status is not None else None, _stream_ptr()))
    return out


def embedding_col(indices: torch.Tensor, matrix: torch.Tensor, scales: torch.Tensor | None = None, vocab: int | None = None,
                  status: torch.Tensor | None = None) -> torch.Tensor:
    """out[i, d] = M[d, indices[i]] for M [dim, vocab_stride] in float16, or int8 with float16 scales [dim / 32, scale_stride]."""
    dim, vstride = matrix.shape
    vocab = vstride if vocab is None else vocab
    fmt = 0 if matrix.dtype == torch.float16 else 1
    ld = (dim + 3) // 4 * 4
    out = torch.zeros((indices.numel(), ld), dtype=torch.float32, device=matrix.device)
    L.check(L.lib().cutb_embedding_col(fmt, indices.data_ptr(), matrix.data_ptr(), scales.data_ptr() if scales is not None else None,
                                       out.data_ptr(), indices.numel(), dim, vocab, vstride,
                                       scales.shape[1] if scales is not None else vstride, ld,
                                       status.data_ptr() if status is not None else None, _stream_ptr()))
    return out


def embedding_blocks(indices: torch.Tensor, raw: torch.Tensor, fmt: int, rows: int, cols: int,
                     status: torch.Tensor | None = None) -> torch.Tensor:
    """out[i, :] = dequant(row indices[i]) of a table kept as raw GGUF blocks (rows x cols weights)."""
    out = torch.empty((indices.numel(), cols), dtype=torch.float32, device=raw.device)
    L.check(L.lib().cutb_embedding_blocks(fmt, indices.data_ptr(), raw.data_ptr(), out.data_ptr(), indices.numel(), rows, cols, cols,
                                          status.data_ptr() if status is not None else None, _stream_ptr()))
    return out


def requant_q8_0_blocks(raw: torch.Tensor, fmt: int, rows: int, cols: int) -> torch.Tensor:
    """Raw blocks of any dequantisable format -> Q8_0 GGUF blocks (uint8, rows * cols / 32 * 34 bytes)."""
    out = torch.empty(rows * (cols // 32) * 34, dtype=torch.uint8, device=raw.device)
    L.check(L.lib().cutb_requant_q8_0_blocks(fmt, raw.data_ptr(), raw.numel() * raw.element_size(), out.data_ptr(), rows, cols,
                                             _stream_ptr()))
    return out


def argreduce(values: torch.Tensor, is_max: bool = True) -> torch.Tensor:
    """Index of the maximum / minimum as a one-element float tensor (the reference's output type and tie rule)."""
    out = torch.empty(1, dtype=torch.float32, device=values.device)
    L.check(L.lib().cutb_argreduce(1 if is_max else 0, values.data_ptr(), out.data_ptr(), values.numel(), _stream_ptr()))
    return out


# ---- decode-step attention ----
def _kv_dtype(cache: torch.Tensor) -> int:
    if cache.dtype == torch.float16:
        return L.F16
    if cache.dtype == torch.float32:
        return L.F32
    raise RuntimeError("KV cache must be float32 or float16")


def rope_kv_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, params: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor,
                  k_cache: torch.Tensor, v_cache: torch.Tensor, head_dim: int, q_out: torch.Tensor | None = None,
                  status: torch.Tensor | None = None) -> torch.Tensor:
    """Half-split RoPE of q and k at params[0]; roped k and v go to row params[0] of the caches
    ([max_seq, ld]); returns the roped q.  params: int32/uint32 device tensor {pos, seqLen}."""
    if q_out is None:
        q_out = torch.empty_like(q)
    L.check(L.lib().cutb_rope_kv_write(_kv_dtype(k_cache), q.data_ptr(), k.data_ptr(), v.data_ptr(), params.data_ptr(),
                                       cos_t.data_ptr(), sin_t.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), q_out.data_ptr(),
                                       q.numel(), k.numel(), head_dim, k_cache.stride(0), k_cache.shape[0],
                                       status.data_ptr() if status is not None else None, _stream_ptr()))
    return q_out


def attention_workspace(n_heads: int, n_kv_heads: int, head_dim: int, max_seq: int, device) -> torch.Tensor:
    """Zeroed scratch for attention_decode (its first 256 bytes are arrival counters that every launch leaves zero)."""
    n = int(L.lib().cutb_attention_workspace_bytes(n_heads, n_kv_heads, head_dim, max_seq))
    return torch.zeros(n, dtype=torch.uint8, device=device)


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, params: torch.Tensor, n_heads: int,
                     n_kv_heads: int, head_dim: int, workspace: torch.Tensor, out: torch.Tensor | None = None,
                     scale: float | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped-query attention of one roped query [n_heads * head_dim] over rows [0, params[1]) of the caches."""
    if out is None:
        out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=q.device)
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    L.check(L.lib().cutb_attention_decode(_kv_dtype(k_cache), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), params.data_ptr(),
                                          out.data_ptr(), n_heads, n_kv_heads, head_dim, k_cache.stride(0), k_cache.shape[0],
                                          scale, workspace.data_ptr(), workspace.numel(),
                                          status.data_ptr() if status is not None else None, _stream_ptr()))
    return out


def rope_attention_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, params: torch.Tensor, cos_t: torch.Tensor,
                          sin_t: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int, n_kv_heads: int,
                          head_dim: int, workspace: torch.Tensor, out: torch.Tensor | None = None, scale: float | None = None,
                          status: torch.Tensor | None = None) -> torch.Tensor:
    """rope_kv_write + attention_decode in one call (one launch where the cluster kernel applies)."""
    if out is None:
        out = torch.empty(n_heads * head_dim, dtype=torch.float32, device=q.device)
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    L.check(L.lib().cutb_rope_attention_decode(_kv_dtype(k_cache), q.data_ptr(), k.data_ptr(), v.data_ptr(), params.data_ptr(),
                                               cos_t.data_ptr(), sin_t.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                               out.data_ptr(), n_heads, n_kv_heads, head_dim, k_cache.stride(0), k_cache.shape[0],
                                               scale, workspace.data_ptr(), workspace.numel(),
                                               status.data_ptr() if status is not None else None, _stream_ptr()))
    return out


# ---- prefill (a batch of prompt tokens) ----
def batched_kv_write(k_in: torch.Tensor, v_in: torch.Tensor, positions: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor,
                     k_cache: torch.Tensor, v_cache: torch.Tensor, head_dim: int, status: torch.Tensor | None = None) -> None:
    """k_cache[positions[i]] = RoPE(k_in[i]), v_cache[positions[i]] = v_in[i]; k_in / v_in are [T, kv_dim] views (any row stride)."""
    L.check(L.lib().cutb_batched_kv_write(_kv_dtype(k_cache), k_in.data_ptr(), v_in.data_ptr(), k_in.stride(0), v_in.stride(0),
                                          positions.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), k_cache.data_ptr(),
                                          v_cache.data_ptr(), k_in.shape[0], k_in.shape[1], head_dim, k_cache.stride(0),
                                          k_cache.shape[0], status.data_ptr() if status is not None else None, _stream_ptr()))


def batched_attention(q_in: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor, cos_t: torch.Tensor,
                      sin_t: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, out: torch.Tensor | None = None,
                      scale: float | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """out[i] = attention of RoPE(q_in[i]) over cache rows [0, positions[i]]; q_in is a [T, n_heads * head_dim] view."""
    T = q_in.shape[0]
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=torch.float32, device=q_in.device)
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    L.check(L.lib().cutb_batched_attention(_kv_dtype(k_cache), q_in.data_ptr(), q_in.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                                           positions.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), out.data_ptr(), out.stride(0), T,
                                           n_heads, n_kv_heads, head_dim, k_cache.stride(0), k_cache.shape[0], scale,
                                           status.data_ptr() if status is not None else None, _stream_ptr()))
    return out


def glu_pairs(x: torch.Tensor, unary_op: int = 133, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, i] = unary(x[r, 2i]) * x[r, 2i + 1] (SiLU by default)."""
    rows, cols = x.shape
    if out is None:
        out = torch.empty((rows, cols // 2), dtype=torch.float32, device=x.device)
    L.check(L.lib().cutb_glu_pairs(x.data_ptr(), out.data_ptr(), rows, cols // 2, x.stride(0), out.stride(0), unary_op, _stream_ptr()))
    return out

