"""Seeded synthetic inputs in the GGUF block formats of the quantized-matmul path.

No model file, tokenizer or dataset is available offline, so every test and the
benchmark build their weights here from a seed, with the block layouts the
reference's loader parses (interface/loader/gguf/gguf_types.hpp:109-150,
gguf_reader.cpp:541-572, 668-724, 826-850) and the value distributions of the
benchmark configurations:

  Q8_0  34-byte blocks: f16 d = |N(0, 0.02)| / 127, then 32 int8 ~ U[-127, 127]
  Q4_0  18-byte blocks: f16 d = |N(0, 0.02)| / 8, then 16 bytes; byte j holds
        element j in the low and element j + 16 in the high nibble, U[0, 15]
  Q4_K  144-byte super-blocks of 256: f16 d, f16 dmin = |N(0, 0.01)|, 12 bytes
        of packed 6-bit (scale, min) pairs ~ U[0, 63], 128 bytes of nibbles
  Q5_K  176-byte super-blocks: the Q4_K header, 32 bytes of fifth bits, 128
        bytes of nibbles (gguf_reader.cpp:726-772); uniform random bits
  Q6_K  210-byte super-blocks: 128 bytes of low nibbles, 64 bytes of 2-bit high
        parts, 16 int8 scales ~ U[-128, 127], f16 d (gguf_reader.cpp:774-824)
  Q4_1  20-byte blocks: f16 scale, f16 minimum, 16 bytes of nibbles; Q5_0  22-byte blocks: f16
        scale, 32 fifth bits, 16 bytes of nibbles (the loader's remaining 32-weight formats)
  BF16  the upper halves of N(0, 1) float32 values, some replaced by
        infinities, NaNs, zeros and subnormals

fp16 conversions round to nearest even and keep subnormals (numpy's astype),
which matters: a third of the Q8_0 scales above are fp16 subnormals.
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_0, Q4_K, Q5_K, Q6_K, BF16, Q4_1, Q5_0 = 0, 1, 2, 3, 4, 5, 6, 7  # from Q5_K on: dequant operator only
FMT_NAMES = {Q8_0: "Q8_0", Q4_0: "Q4_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", BF16: "BF16", Q4_1: "Q4_1", Q5_0: "Q5_0"}
BLOCK_ELEMS = {Q8_0: 32, Q4_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256, BF16: 1, Q4_1: 32, Q5_0: 32}
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18, Q4_K: 144, Q5_K: 176, Q6_K: 210, BF16: 2, Q4_1: 20, Q5_0: 22}


def row_bytes(fmt: int, K: int) -> int:
    be = BLOCK_ELEMS[fmt]
    return (K + be - 1) // be * BLOCK_BYTES[fmt]


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def pack_q4k_scales(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """Pack 8 six-bit scales and 8 six-bit mins ([..., 8] uint8 each) into the 12
    bytes that get_scale_min_k4 (gguf_reader.cpp:668-676) unpacks."""
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (m[..., 0:4] & 63) | ((m[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0xF) | ((m[..., 4:8] & 0xF) << 4)
    return out


def make_weights(fmt: int, N: int, K: int, seed: int) -> np.ndarray:
    """N rows of GGUF blocks along K, as a flat uint8 array of N * row_bytes."""
    rng = _rng(seed)
    be = BLOCK_ELEMS[fmt]
    if K % be:
        raise ValueError(f"K={K} is not a multiple of the {FMT_NAMES[fmt]} block ({be})")
    nb = N * (K // be)
    blocks = np.empty((nb, BLOCK_BYTES[fmt]), dtype=np.uint8)
    if fmt == Q8_0:
        d = (np.abs(rng.normal(0.0, 0.02, nb)) / 127.0).astype(np.float32).astype(np.float16)
        q = rng.integers(-127, 128, size=(nb, 32), dtype=np.int16).astype(np.int8)
        blocks[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        blocks[:, 2:34] = q.view(np.uint8)
    elif fmt == Q4_0:
        d = (np.abs(rng.normal(0.0, 0.02, nb)) / 8.0).astype(np.float32).astype(np.float16)
        nib = rng.integers(0, 16, size=(nb, 32), dtype=np.uint8)
        blocks[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        blocks[:, 2:18] = nib[:, 0:16] | (nib[:, 16:32] << 4)
    elif fmt == Q4_K:
        d = np.abs(rng.normal(0.0, 0.01, nb)).astype(np.float32).astype(np.float16)
        dmin = np.abs(rng.normal(0.0, 0.01, nb)).astype(np.float32).astype(np.float16)
        sc = rng.integers(0, 64, size=(nb, 8), dtype=np.uint8)
        m = rng.integers(0, 64, size=(nb, 8), dtype=np.uint8)
        nib = rng.integers(0, 16, size=(nb, 4, 2, 32), dtype=np.uint8)
        blocks[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        blocks[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
        blocks[:, 4:16] = pack_q4k_scales(sc, m)
        blocks[:, 16:144] = (nib[:, :, 0, :] | (nib[:, :, 1, :] << 4)).reshape(nb, 128)
    elif fmt == Q5_K:
        d = np.abs(rng.normal(0.0, 0.01, nb)).astype(np.float32).astype(np.float16)
        dmin = np.abs(rng.normal(0.0, 0.01, nb)).astype(np.float32).astype(np.float16)
        blocks[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        blocks[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
        blocks[:, 4:16] = pack_q4k_scales(rng.integers(0, 64, size=(nb, 8), dtype=np.uint8),
                                          rng.integers(0, 64, size=(nb, 8), dtype=np.uint8))
        blocks[:, 16:176] = rng.integers(0, 256, size=(nb, 160), dtype=np.uint8)
    elif fmt == Q6_K:
        d = np.abs(rng.normal(0.0, 0.002, nb)).astype(np.float32).astype(np.float16)
        blocks[:, 0:208] = rng.integers(0, 256, size=(nb, 208), dtype=np.uint8)
        blocks[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
    elif fmt == Q4_1:
        d = (np.abs(rng.normal(0.0, 0.02, nb)) / 8.0).astype(np.float32).astype(np.float16)
        m = rng.normal(0.0, 0.02, nb).astype(np.float32).astype(np.float16)
        nib = rng.integers(0, 16, size=(nb, 32), dtype=np.uint8)
        blocks[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        blocks[:, 2:4] = m.view(np.uint8).reshape(nb, 2)
        blocks[:, 4:20] = nib[:, 0:16] | (nib[:, 16:32] << 4)
    elif fmt == Q5_0:
        d = (np.abs(rng.normal(0.0, 0.02, nb)) / 16.0).astype(np.float32).astype(np.float16)
        blocks[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        blocks[:, 2:22] = rng.integers(0, 256, size=(nb, 20), dtype=np.uint8)
    elif fmt == BF16:
        x = rng.normal(0.0, 1.0, nb).astype(np.float32)
        bits = (x.view(np.uint32) >> 16).astype(np.uint16)
        special = np.array([0x7F80, 0xFF80, 0x7FC0, 0x0000, 0x8000, 0x0001, 0x807F, 0x7F7F], dtype=np.uint16)
        idx = rng.integers(0, nb, size=min(nb, 64))
        bits[idx] = special[rng.integers(0, special.size, size=idx.size)]
        blocks[:, 0:2] = bits.view(np.uint8).reshape(nb, 2)
    else:
        raise ValueError(f"unknown format {fmt}")
    return blocks.reshape(-1)


def make_activations(M: int, K: int, seed: int, dtype=np.float32) -> np.ndarray:
    """[M, K] activations ~ N(0, 1) in float32 or float16."""
    a = _rng(seed).normal(0.0, 1.0, size=(M, K)).astype(np.float32)
    return a.astype(dtype)
