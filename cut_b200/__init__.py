"""B200-native GGUF quantized matmul behind CUT's operator API.

The product is libcutb.so (include/cutb.h): hand-written sm_100a kernels behind
a C ABI.  This package builds it, loads it, and offers a thin torch harness for
tests and measurements.
"""
from . import synth  # noqa: F401

__all__ = ["synth"]
