"""A small GGUF v3 writer: metadata scalars / strings and 1-D / 2-D tensors of raw bytes.

What `cut_b200/csrc/host/gguf_upload.cpp` (GGUFFile) and the reference's reader
(interface/loader/gguf/gguf_reader.cpp:15-58, 268-291) parse: magic, version, counts, metadata pairs
{key, value type, value}, the tensor directory {name, n_dims, dims innermost first, ggml type, offset}, then
the data section at the next multiple of the alignment, every tensor offset aligned.  Used to turn synthetic
weights into model files for the C++ runner; not a general exporter (no arrays, no tokenizer).
"""
from __future__ import annotations

import struct

import numpy as np

GGML_TYPE = {"F32": 0, "F16": 1, "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q8_0": 8, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14, "BF16": 30}
_U32, _F32, _STR = 4, 6, 8  # GGUF metadata value types


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str, metadata: dict, tensors: list, alignment: int = 32) -> None:
    """metadata: {key: int | float | str}; tensors: [(name, ggml type name, dims outermost first, raw bytes array)]."""
    head = bytearray(struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(metadata)))
    for key, val in metadata.items():
        head += _s(key)
        if isinstance(val, str):
            head += struct.pack("<I", _STR) + _s(val)
        elif isinstance(val, float):
            head += struct.pack("<If", _F32, val)
        else:
            head += struct.pack("<II", _U32, int(val))
    offset, offsets = 0, []
    for name, tname, dims, raw in tensors:
        head += _s(name) + struct.pack("<I", len(dims))
        for d in reversed(dims):  # innermost first
            head += struct.pack("<Q", int(d))
        head += struct.pack("<IQ", GGML_TYPE[tname], offset)
        offsets.append(offset)
        offset = (offset + np.asarray(raw).nbytes + alignment - 1) // alignment * alignment
    start = (len(head) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (start - len(head)))
        pos = 0
        for (_, _, _, raw), off in zip(tensors, offsets):
            f.write(b"\0" * (off - pos))
            data = np.ascontiguousarray(raw).tobytes()
            f.write(data)
            pos = off + len(data)
