"""Minimal GGUF v3 writer for feeding synthetic tensors to the reference's reader.

TEST INFRASTRUCTURE ONLY.  Writes the header the reference parses
(interface/loader/gguf/gguf_reader.cpp:15-58, 281-291): magic, version 3,
tensor count, zero metadata pairs, then per tensor {name, n_dims, dims (inner
first), ggml type, offset}; tensor data starts at the next multiple of 32 bytes
and every tensor offset is 32-byte aligned.
"""
from __future__ import annotations

import struct

import numpy as np

GGML_TYPE = {"F32": 0, "F16": 1, "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q8_0": 8, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14, "BF16": 30}


def write_gguf(path: str, tensors: list[tuple[str, str, tuple[int, int], np.ndarray]]) -> None:
    """tensors: (name, ggml type name, (rows, cols), raw uint8 bytes)."""
    head = bytearray()
    head += struct.pack("<IIQQ", 0x46554747, 3, len(tensors), 0)
    offset = 0
    offsets = []
    for name, tname, (rows, cols), raw in tensors:
        nm = name.encode()
        head += struct.pack("<Q", len(nm)) + nm
        head += struct.pack("<I", 2) + struct.pack("<QQ", cols, rows)
        head += struct.pack("<IQ", GGML_TYPE[tname], offset)
        offsets.append(offset)
        offset = (offset + raw.nbytes + 31) // 32 * 32
    data_start = (len(head) + 31) // 32 * 32
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (data_start - len(head)))
        pos = 0
        for (name, tname, shape, raw), off in zip(tensors, offsets):
            f.write(b"\0" * (off - pos))
            f.write(np.ascontiguousarray(raw).tobytes())
            pos = off + raw.nbytes
