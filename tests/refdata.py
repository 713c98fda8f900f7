"""Inputs of the reference's own known-answer tests, regenerated bit-for-bit.

The reference's tests build their data in code; these helpers restate those
generators so the replayed cases see identical inputs:
  * generateTestData<float>(count, 42): std::mt19937 + uniform_real(0.1, 10)
    (tests/harness/OpRefs.h:241-266);
  * the model-geometry tests' uniform_real(-1, 1) (tests/runtime/RuntimeTests.cpp:2865-2868);
  * packNibbles (OpRefs.h:178-180) and the truncating f32_to_f16 (OpRefs.h:164-177,
    taken from the CPU checker).
tests/golden/golden.npz pins the first values of both streams as produced by a
C++ program using the same standard-library calls.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def mt19937_uniform(lo: float, hi: float, seed: int, count: int) -> np.ndarray:
    """libstdc++ uniform_real_distribution<float>(lo, hi) over std::mt19937(seed)."""
    raw = np.random.RandomState(seed)._bit_generator.random_raw(count)
    can = raw.astype(np.float32) / np.float32(4294967296.0)
    can = np.where(can >= 1.0, np.nextafter(np.float32(1), np.float32(0)), can).astype(np.float32)
    return (can * (np.float32(hi) - np.float32(lo)) + np.float32(lo)).astype(np.float32)


def generate_test_data(count: int, seed: int = 42) -> np.ndarray:
    return mt19937_uniform(0.1, 10.0, seed, count)


def f16_trunc(values) -> np.ndarray:
    return np.array([O.f32_to_f16_trunc(float(v)) for v in np.asarray(values, dtype=np.float32).reshape(-1)],
                    dtype=np.uint16)


def pack_nibbles(lo, hi):
    return (np.asarray(lo, dtype=np.uint8) & 0xF) | ((np.asarray(hi, dtype=np.uint8) & 0xF) << 4)


def pad4(n: int) -> int:
    return (n + 3) & ~3


# --- the reference's quantized-matmul cases (tests/harness/OpRegistry.h:1995-2192) ---
def case_q8(M, K, N, a_mode):
    """Returns (A[M,K] f32, B[K,N] int8, scale floats [K/32,N], scale f16 bits)."""
    if a_mode == "ones":
        A = np.ones((M, K), dtype=np.float32)
    else:
        A = generate_test_data(M * K).reshape(M, K)
    i = np.arange(K * N, dtype=np.int64)
    B = ((i * 7 + 3) % 21 - 10).astype(np.int8).reshape(K, N)
    sf = (np.float32(0.1) + np.float32(0.05) * np.arange((K // 32) * N, dtype=np.float32)).astype(np.float32)
    return A, B, sf.reshape(K // 32, N), f16_trunc(sf).reshape(K // 32, N)


def case_q4(M, K, N, a_mode):
    """Returns (A, packedB [K,N/2] u8, nibbles [K,N], scale floats, scale f16 bits)."""
    if a_mode == "ones":
        A = np.ones((M, K), dtype=np.float32)
    else:
        A = generate_test_data(M * K).reshape(M, K)
    i = np.arange(K * N, dtype=np.int64)
    nib = ((i * 7 + 3) % 16).astype(np.uint8).reshape(K, N)
    packed = pack_nibbles(nib[:, 0::2], nib[:, 1::2])
    sf = (np.float32(0.1) + np.float32(0.05) * np.arange((K // 32) * N, dtype=np.float32)).astype(np.float32)
    return A, packed, nib, sf.reshape(K // 32, N), f16_trunc(sf).reshape(K // 32, N)
