"""Launches the reference's own CUDA matmul kernels (cubins built by build_ref_cuda.py) on torch CUDA tensors.

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
