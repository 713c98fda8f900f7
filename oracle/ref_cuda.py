"""Launches the reference's own CUDA kernels of this path (cubins built by build_ref_cuda.py) on torch CUDA tensors.

TEST / BASELINE INFRASTRUCTURE ONLY: the GPU-side checker of the plane-layout kernels and the reference-GPU
baseline of bench.py.  Each kernel is the reference's `cut_main(dataA, packedB, scalesB, dataD, dataC, push)` with
its launch geometry: the K-parallel mat-vecs run (32, 8) threads per 8 output columns and one grid row per
activation row (operators/impl/matmul/MatMulQ4GemvKPar8.cu:8-24, MatMulQ8GemvKPar8.cu:11-27); the tensor-core tiled
kernels run 128 threads per 32 x 32 output tile (MatMulQ4CoopMatTiled.cu:7-30).  Operands are the reference's
run-time layout: fp32 A [M, strideA], int8 [K, strideB] or nibbles [K, strideB bytes], fp16 scales
[K / 32, scaleStride], fp32 C [M, strideC]; no fusion (specialisation constants 0).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
CUBIN_DIR = os.path.join(_HERE, "_ref", "cuda")
_modules: dict = {}


class _Push(C.Structure):
    _fields_ = [("M", C.c_uint32), ("K", C.c_uint32), ("N", C.c_uint32), ("strideA", C.c_uint32), ("strideB", C.c_uint32),
                ("strideC", C.c_uint32), ("scaleStride", C.c_uint32)]


def have(kernel: str) -> bool:
    return os.path.exists(os.path.join(CUBIN_DIR, kernel + ".cubin"))


def _function(kernel: str):
    import torch
    from cuda.bindings import driver

    key = (kernel, torch.cuda.current_device())
    if key not in _modules:
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # the primary context is current on this thread
        with open(os.path.join(CUBIN_DIR, kernel + ".cubin"), "rb") as f:
            image = f.read()
        err, mod = driver.cuModuleLoadData(image)
        if int(err) != 0:
            raise RuntimeError(f"cuModuleLoadData({kernel}): {err}")
        err, fn = driver.cuModuleGetFunction(mod, b"cut_main")
        if int(err) != 0:
            raise RuntimeError(f"cuModuleGetFunction({kernel}): {err}")
        _modules[key] = (mod, fn)
    return _modules[key][1]


def launch(kernel: str, A, B, S, Cout, M: int, K: int, N: int, *, stride_a: int, stride_b: int, stride_c: int, scale_stride: int) -> None:
    """Enqueues one launch of `kernel` on torch's current stream."""
    import torch
    from cuda.bindings import driver

    fn = _function(kernel)
    if "GemvKPar8" in kernel:
        if N % 8 or stride_b % 4 or scale_stride % 4:
            raise ValueError("the K-parallel mat-vec reads 8 columns per group through 4-byte / 4-scale loads")
        grid, block = ((N + 7) // 8, M, 1), (32, 8, 1)
    else:
        if K % 16 or N % 32:
            raise ValueError("the tiled kernel needs K % 16 == 0 and N % 32 == 0")
        grid, block = (N // 32, (M + 31) // 32, 1), (128, 1, 1)
    ptrs = [C.c_void_p(t.data_ptr()) for t in (A, B, S, Cout, Cout)]  # D is not read without a binary fusion
    push = _Push(M, K, N, stride_a, stride_b, stride_c, scale_stride)
    args = (C.c_void_p * 6)(*[C.addressof(p) for p in ptrs], C.addressof(push))
    (err,) = driver.cuLaunchKernel(fn, *grid, *block, 0, torch.cuda.current_stream().cuda_stream, C.addressof(args), 0)
    if int(err) != 0:
        raise RuntimeError(f"cuLaunchKernel({kernel}): {err}")


def _launch_raw(kernel: str, grid, block, tensors, push: C.Structure) -> None:
    import torch
    from cuda.bindings import driver

    fn = _function(kernel)
    ptrs = [C.c_void_p(t.data_ptr()) for t in tensors]
    args = (C.c_void_p * (len(ptrs) + 1))(*[C.addressof(p) for p in ptrs], C.addressof(push))
    (err,) = driver.cuLaunchKernel(fn, *grid, *block, 0, torch.cuda.current_stream().cuda_stream, C.addressof(args), 0)
    if int(err) != 0:
        raise RuntimeError(f"cuLaunchKernel({kernel}): {err}")


class _AttnPush(C.Structure):
    _fields_ = [("nHeads", C.c_uint32), ("nKvHeads", C.c_uint32), ("headDim", C.c_uint32), ("kvDim", C.c_uint32),
                ("alignedKvDim", C.c_uint32), ("nRep", C.c_uint32), ("scale", C.c_float)]


def attention(kv_half: bool, q, k_cache, v_cache, params, out, n_heads: int, n_kv_heads: int, head_dim: int, scale: float) -> None:
    """The reference's decode attention (operators/impl/attention/Attention.cu: one 256-thread block per query head,
    scores in a 2048-entry shared array, so seqLen <= 2048 and head_dim <= 128).  Caches are [rows, alignedKvDim]."""
    if head_dim > 128:
        raise ValueError("the reference kernel holds one query head of at most 128 elements")
    kv_dim = n_kv_heads * head_dim
    push = _AttnPush(n_heads, n_kv_heads, head_dim, kv_dim, k_cache.stride(0), n_heads // n_kv_heads, scale)
    _launch_raw("Attention_f16" if kv_half else "Attention", (n_heads, 1, 1), (256, 1, 1), (q, k_cache, v_cache, params, out), push)


class _RopePush(C.Structure):
    _fields_ = [("qDim", C.c_uint32), ("kvDim", C.c_uint32), ("headDim", C.c_uint32), ("halfDim", C.c_uint32), ("alignedKvDim", C.c_uint32)]


def rope_kv_write(kv_half: bool, q, k, v, params, cos_t, sin_t, k_cache, v_cache, q_roped, q_dim: int, kv_dim: int, head_dim: int) -> None:
    """The reference's fused RoPE + KV-cache write (operators/impl/attention/FusedRoPEKVWrite.cu: one thread per element
    of q, k and v, 256 per block)."""
    push = _RopePush(q_dim, kv_dim, head_dim, head_dim // 2, k_cache.stride(0))
    total = q_dim + 2 * kv_dim
    _launch_raw("FusedRoPEKVWrite_f16" if kv_half else "FusedRoPEKVWrite", ((total + 255) // 256, 1, 1), (256, 1, 1),
                (q, k, v, params, cos_t, sin_t, k_cache, v_cache, q_roped), push)


class _DequantPush(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("cols", C.c_uint32), ("outputStride", C.c_uint32)]


def dequant(kernel: str, raw, out, rows: int, cols: int) -> None:
    """The reference's dequant operators (operators/impl/dequant/DequantQ4K.cu, DequantQ5K.cu, DequantQ6K.cu, DequantBF16.cu:
    256 x 1 threads, one element each)."""
    _launch_raw(kernel, ((cols + 255) // 256, rows, 1), (256, 1, 1), (raw, out), _DequantPush(rows, cols, out.stride(0)))


def dequant_q4k(raw, out, rows: int, cols: int) -> None:
    dequant("DequantQ4K", raw, out, rows, cols)


class _RmsPush(C.Structure):
    _fields_ = [("dim", C.c_uint32), ("alignedDim", C.c_uint32), ("eps", C.c_float)]


def rmsnorm(x, weight, out, rows: int, dim: int, eps: float) -> None:
    """The reference's RMSNorm (operators/impl/rmsnorm/RMSNorm.cu: one 256-thread block per row, fp32)."""
    _launch_raw("RMSNorm", (1, rows, 1), (256, 1, 1), (x, weight, out), _RmsPush(dim, x.stride(0) if x.dim() == 2 else (dim + 3) // 4 * 4, eps))


class _ArgPush(C.Structure):
    _fields_ = [("numElements", C.c_uint32)]


def argmax(v, out, n: int) -> None:
    """The reference's arg-max (operators/impl/reduce/ReduceArg.cu: one block of 256 threads, strided scan + tree)."""
    _launch_raw("ReduceArgmax", (1, 1, 1), (256, 1, 1), (v, out), _ArgPush(n))


class _BkvPush(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("batchSize", "kvDim", "alignedKvDim", "headDim", "halfDim", "kStride", "vStride", "kOffset", "vOffset")]


def batched_kv_write(kv_half: bool, k_in, v_in, k_cache, v_cache, positions, cos_t, sin_t, batch: int, kv_dim: int, head_dim: int,
                     k_stride: int, v_stride: int, k_offset: int, v_offset: int) -> None:
    """The reference's batched RoPE + cache write (operators/impl/attention/BatchedKVCacheWrite.cu: one block per token)."""
    push = _BkvPush(batch, kv_dim, k_cache.stride(0), head_dim, head_dim // 2, k_stride, v_stride, k_offset, v_offset)
    _launch_raw("BatchedKVCacheWrite_f16" if kv_half else "BatchedKVCacheWrite", (1, batch, 1), (256, 1, 1),
                (k_in, v_in, k_cache, v_cache, positions, cos_t, sin_t), push)


class _BattPush(C.Structure):
    _fields_ = [("batchSize", C.c_uint32), ("nHeads", C.c_uint32), ("nKvHeads", C.c_uint32), ("headDim", C.c_uint32),
                ("alignedKvDim", C.c_uint32), ("nRep", C.c_uint32), ("scale", C.c_float), ("halfDim", C.c_uint32),
                ("qStride", C.c_uint32), ("qOffset", C.c_uint32)]


def batched_attention(kv_half: bool, q_in, k_cache, v_cache, positions, cos_t, sin_t, out, batch: int, n_heads: int, n_kv_heads: int,
                      head_dim: int, scale: float, q_stride: int, q_offset: int) -> None:
    """The reference's batched prefill attention (operators/impl/attention/BatchedAttentionReadCache.cu: one block per
    (query head, token), positions < 2048, head_dim <= 128; output [batch, nHeads * headDim])."""
    if head_dim > 128:
        raise ValueError("the reference kernel holds one query head of at most 128 elements")
    push = _BattPush(batch, n_heads, n_kv_heads, head_dim, k_cache.stride(0), n_heads // n_kv_heads, scale, head_dim // 2, q_stride, q_offset)
    _launch_raw("BatchedAttentionReadCache_f16" if kv_half else "BatchedAttentionReadCache", (n_heads, batch, 1), (256, 1, 1),
                (q_in, k_cache, v_cache, positions, cos_t, sin_t, out), push)
