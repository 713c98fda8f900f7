"""Builds libcutb.so (the C ABI + sm_100a kernels) in-tree with nvcc.

nvcc cross-compiles for sm_100a without a GPU, so this runs anywhere the CUDA
toolkit is installed.  The library lands next to this file so that it travels
with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcutb.so")
SOURCES = ["cabi.cu", "common.cu", "qgemv_blocks.cu", "qmatmul_generic.cu", "dequant.cu", "transpose_q4.cu",
           "qgemm_tc.cu", "qgemm_skinny.cu", "repack.cu", "layer_ops.cu", "attention.cu", "attention_prefill.cu", "qgemv_planes.cu"]
HEADERS = ["common.cuh", "kernels.h", "qgemm_tc_common.cuh", os.path.join("..", "..", "include", "cutb.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu into an object (only the stale ones) and link libcutb.so."""
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    objs, procs = [], []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", s, "-o", o] + (["-Xptxas", "-v"] if verbose else [])
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose:
            print(out)
    if force or procs or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    return LIB


HOST_LIB = os.path.join(HERE, "libcut_host.so")
HOST_SOURCES = ["cut_api.cpp", "b200_compute.cpp", "gguf_upload.cpp", "llama_runner.cpp", "host_cabi.cpp"]


def _cuda_home() -> str:
    return os.path.dirname(os.path.dirname(_nvcc()))


def build_host(force: bool = False) -> str:
    """Compile the C++ host API (csrc/host) into libcut_host.so on top of libcutb.so."""
    build(force=force)
    hdir = os.path.join(CSRC, "host")
    srcs = [os.path.join(hdir, f) for f in HOST_SOURCES]
    deps = srcs + [os.path.join(hdir, "cut_api.h"), os.path.join(hdir, "gguf_upload.h"),
                   os.path.join(CSRC, "..", "..", "include", "cutb.h"), LIB]
    if force or _stale(HOST_LIB, deps):
        cuda = _cuda_home()
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-o", HOST_LIB, *srcs, f"-I{cuda}/include",
               f"-L{cuda}/lib64", f"-L{HERE}", "-lcutb", "-lcudart_static", "-ldl", "-lrt", "-lpthread",
               "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"host build failed:\n{r.stdout}{r.stderr}")
    return HOST_LIB


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_host(force="--force" in sys.argv))
