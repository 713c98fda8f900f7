"""Compiles the reference's own CUDA kernels of this path for sm_100a, as its backend does at run time.

TEST / BASELINE INFRASTRUCTURE ONLY.  The reference hands `#include "cut_cuda_prelude.cuh"` + a kernel's .cu text
to NVRTC with its headers by name and `--std=c++17` (core/backends/cuda/CudaContainers.cpp:94-222).  This script
does the same from the sources where they lie in the reference tree (nothing is copied into this repository) and
writes one cubin per kernel into oracle/_ref/cuda/ -- the checker the plane-layout kernels are compared with on the
GPU, and the reference-GPU baseline `bench.py` times beside them.  NVRTC needs no GPU.

    python oracle/build_ref_cuda.py /path/to/reference [out_dir]
"""
from __future__ import annotations

import os
import sys

# cubin name -> (kernel source in the reference tree, extra -D options: the per-variant defines of its kernel table)
SOURCES = {
    "MatMulQ4GemvKPar8": ("operators/impl/matmul/MatMulQ4GemvKPar8.cu", []),
    "MatMulQ8GemvKPar8": ("operators/impl/matmul/MatMulQ8GemvKPar8.cu", []),
    "MatMulQ4CoopMatTiled": ("operators/impl/matmul/MatMulQ4CoopMatTiled.cu", []),
    "MatMulQ8CoopMatTiled": ("operators/impl/matmul/MatMulQ8CoopMatTiled.cu", []),
    "Attention": ("operators/impl/attention/Attention.cu", []),
    "Attention_f16": ("operators/impl/attention/Attention.cu", ["-DCUT_DTYPE_INPUT_IS_HALF=1"]),
    "FusedRoPEKVWrite": ("operators/impl/attention/FusedRoPEKVWrite.cu", []),
    "FusedRoPEKVWrite_f16": ("operators/impl/attention/FusedRoPEKVWrite.cu", ["-DCUT_DTYPE_INPUT_IS_HALF=1"]),
    "DequantQ4K": ("operators/impl/dequant/DequantQ4K.cu", []),
    "DequantQ5K": ("operators/impl/dequant/DequantQ5K.cu", []),
    "DequantQ6K": ("operators/impl/dequant/DequantQ6K.cu", []),
    "DequantBF16": ("operators/impl/dequant/DequantBF16.cu", []),
    "RMSNorm": ("operators/impl/rmsnorm/RMSNorm.cu", []),
    "ReduceArgmax": ("operators/impl/reduce/ReduceArg.cu", []),
    "BatchedKVCacheWrite": ("operators/impl/attention/BatchedKVCacheWrite.cu", []),
    "BatchedKVCacheWrite_f16": ("operators/impl/attention/BatchedKVCacheWrite.cu", ["-DCUT_DTYPE_INPUT_IS_HALF=1"]),
    "BatchedAttentionReadCache": ("operators/impl/attention/BatchedAttentionReadCache.cu", []),
    "BatchedAttentionReadCache_f16": ("operators/impl/attention/BatchedAttentionReadCache.cu", ["-DCUT_DTYPE_INPUT_IS_HALF=1"]),
}
KERNELS = list(SOURCES)
HEADERS = {"cut_cuda_prelude.cuh": "operators/runtime/cuda/cut_cuda_prelude.cuh", "ComputeOpsShared.h": "operators/runtime/ComputeOpsShared.h",
           "MatMulCommon.cuh": "operators/impl/matmul/MatMulCommon.cuh", "MatMulCoopMatCommon.cuh": "operators/impl/matmul/MatMulCoopMatCommon.cuh",
           "MatMulQ4Common.cuh": "operators/impl/matmul/MatMulQ4Common.cuh", "MatMulQ8Common.cuh": "operators/impl/matmul/MatMulQ8Common.cuh",
           "AttentionCommon.cuh": "operators/impl/attention/AttentionCommon.cuh", "DequantCommon.cuh": "operators/impl/dequant/DequantCommon.cuh",
           "RMSNormCommon.cuh": "operators/impl/rmsnorm/RMSNormCommon.cuh"}


def build(ref_root: str, out_dir: str) -> list[str]:
    """Returns the cubins written (kernels NVRTC rejects are reported on stderr and skipped)."""
    from cuda.bindings import nvrtc

    def rd(rel: str) -> bytes:
        with open(os.path.join(ref_root, rel), "rb") as f:
            return f.read()

    os.makedirs(out_dir, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    opts = [b"--gpu-architecture=sm_100a", b"--std=c++17", f"-I{cuda_home}/include".encode(), f"-I{cuda_home}/include/cccl".encode()]
    names = [n.encode() for n in HEADERS]
    srcs = [rd(p) for p in HEADERS.values()]
    written = []
    for k in KERNELS:
        rel, defines = SOURCES[k]
        src = b'#include "cut_cuda_prelude.cuh"\n' + rd(rel)
        err, prog = nvrtc.nvrtcCreateProgram(src, b"cut_kernel.cu", len(names), srcs, names)
        if int(err) != 0:
            print(f"build_ref_cuda: nvrtcCreateProgram failed for {k}: {err}", file=sys.stderr)
            continue
        kopts = opts + [d.encode() for d in defines]
        (res,) = nvrtc.nvrtcCompileProgram(prog, len(kopts), kopts)
        if int(res) != 0:
            _, n = nvrtc.nvrtcGetProgramLogSize(prog)
            log = b" " * n
            nvrtc.nvrtcGetProgramLog(prog, log)
            print(f"build_ref_cuda: {k} does not compile here: {log.decode(errors='replace')[:400]}", file=sys.stderr)
            nvrtc.nvrtcDestroyProgram(prog)
            continue
        _, size = nvrtc.nvrtcGetCUBINSize(prog)
        cubin = b" " * size
        nvrtc.nvrtcGetCUBIN(prog, cubin)
        nvrtc.nvrtcDestroyProgram(prog)
        path = os.path.join(out_dir, k + ".cubin")
        with open(path, "wb") as f:
            f.write(cubin)
        written.append(path)
    return written


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REF_ROOT", "")
    out = sys.argv[2] if len(sys.argv) > 2 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "cuda")
    if not root or not os.path.isdir(root):
        raise SystemExit("usage: build_ref_cuda.py <reference tree> [out dir]")
    for p in build(root, out):
        print(p)
