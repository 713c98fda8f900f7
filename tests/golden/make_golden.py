"""Regenerates the golden fixtures in this directory.

Run from the repository root in a container that has the reference checked out
(the fixtures themselves are committed, so the tests never need it):

    python tests/golden/make_golden.py

It (1) builds oracle/_ref/libcutref.so from the reference's unmodified
gguf_reader.cpp, (2) pushes hand-crafted edge-case blocks and seeded random
blocks of Q8_0 / Q4_0 / Q4_K (and Q5_K / Q6_K / BF16, which only the dequant
operator takes) through the reference's GGUFReader and stores the
raw bytes next to the float32 bit patterns and separated planes it returned,
and (3) stores the mt19937 activation vectors of the reference's own tests.
"""
from __future__ import annotations

import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
HERE = os.path.dirname(os.path.abspath(__file__))

from cut_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

# Scale bit patterns worth pinning: +-0, smallest/largest subnormal, smallest
# normal, 1.0, largest finite, negatives.  Inf/NaN scales are left out: the CPU
# reader returns one canonical NaN while a GPU propagates payloads.
EDGE_D = [0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0xBC00, 0x83FF, 0x2E66, 0x0200, 0x1234]


def edge_q8_0() -> np.ndarray:
    blocks = np.zeros((len(EDGE_D) * 2, 34), dtype=np.uint8)
    for i, d in enumerate(EDGE_D):
        for v in range(2):
            b = blocks[2 * i + v]
            b[0:2] = np.array([d], dtype=np.uint16).view(np.uint8)
            q = (np.arange(32) * 8 - 128 + v * 7) if v == 0 else np.array([-128, 127, -1, 0, 1, -127] * 6)[:32]
            b[2:] = q.astype(np.int8).view(np.uint8)
    return blocks.reshape(-1)


def edge_q4_0() -> np.ndarray:
    blocks = np.zeros((len(EDGE_D) * 2, 18), dtype=np.uint8)
    for i, d in enumerate(EDGE_D):
        for v in range(2):
            b = blocks[2 * i + v]
            b[0:2] = np.array([d], dtype=np.uint16).view(np.uint8)
            nib = (np.arange(32) % 16) if v == 0 else np.array([0, 15, 8, 7] * 8)
            b[2:] = (nib[:16] | (nib[16:] << 4)).astype(np.uint8)
    return blocks.reshape(-1)


def edge_q4_k() -> np.ndarray:
    pats = [(0x3C00, 0x0000), (0x3C00, 0x3C00), (0x0001, 0x03FF), (0x03FF, 0x0001), (0x7BFF, 0x0400),
            (0xBC00, 0x2E66), (0x1234, 0x8001), (0x0000, 0x3C00)]
    blocks = np.zeros((len(pats) * 2, 144), dtype=np.uint8)
    for i, (d, dm) in enumerate(pats):
        for v in range(2):
            b = blocks[2 * i + v]
            b[0:2] = np.array([d], dtype=np.uint16).view(np.uint8)
            b[2:4] = np.array([dm], dtype=np.uint16).view(np.uint8)
            if v == 0:
                sc = np.array([63, 0, 1, 32, 33, 47, 48, 63], dtype=np.uint8)
                m = np.array([0, 63, 31, 16, 15, 62, 17, 63], dtype=np.uint8)
            else:
                sc = (np.arange(8) * 9 % 64).astype(np.uint8)
                m = (63 - np.arange(8) * 7).astype(np.uint8)
            b[4:16] = synth.pack_q4k_scales(sc, m)
            qs = (np.arange(128) * (3 + v) % 256).astype(np.uint8)
            b[16:] = qs
    return blocks.reshape(-1)


def edge_q5_k() -> np.ndarray:
    pats = [(0x3C00, 0x0000), (0x3C00, 0x3C00), (0x0001, 0x03FF), (0x7BFF, 0x0400), (0xBC00, 0x2E66), (0x0000, 0x3C00)]
    blocks = np.zeros((len(pats) * 2, 176), dtype=np.uint8)
    for i, (d, dm) in enumerate(pats):
        for v in range(2):
            b = blocks[2 * i + v]
            b[0:2] = np.array([d], dtype=np.uint16).view(np.uint8)
            b[2:4] = np.array([dm], dtype=np.uint16).view(np.uint8)
            sc = np.array([63, 0, 1, 32, 33, 47, 48, 63], dtype=np.uint8) if v == 0 else (np.arange(8) * 9 % 64).astype(np.uint8)
            m = np.array([0, 63, 31, 16, 15, 62, 17, 63], dtype=np.uint8) if v == 0 else (63 - np.arange(8) * 7).astype(np.uint8)
            b[4:16] = synth.pack_q4k_scales(sc, m)
            b[16:48] = (np.arange(32) * (37 + 64 * v) % 256).astype(np.uint8)  # fifth bits: every mask position exercised
            b[48:] = (np.arange(128) * (3 + v) % 256).astype(np.uint8)
    return blocks.reshape(-1)


def edge_q6_k() -> np.ndarray:
    ds = [0x3C00, 0x0001, 0x03FF, 0x7BFF, 0xBC00, 0x0000, 0x2E66, 0x8400]
    blocks = np.zeros((len(ds) * 2, 210), dtype=np.uint8)
    for i, d in enumerate(ds):
        for v in range(2):
            b = blocks[2 * i + v]
            b[0:128] = (np.arange(128) * (5 + 2 * v) % 256).astype(np.uint8)
            b[128:192] = (np.arange(64) * (11 + 4 * v) % 256).astype(np.uint8)
            sc = np.array([-128, 127, -1, 0, 1, 64, -64, 33, 2, -2, 100, -100, 17, -17, 127, -128], dtype=np.int8)
            b[192:208] = (sc if v == 0 else sc[::-1]).view(np.uint8)
            b[208:210] = np.array([d], dtype=np.uint16).view(np.uint8)
    return blocks.reshape(-1)


def edge_bf16() -> np.ndarray:
    # +-0, subnormals, smallest normal, 1, largest finite, +-inf, quiet and signalling NaN payloads
    bits = np.array([0x0000, 0x8000, 0x0001, 0x007F, 0x0080, 0x3F80, 0xBF80, 0x7F7F, 0xFF7F, 0x7F80, 0xFF80, 0x7FC0,
                     0x7FA1, 0xFFFF, 0x4049, 0x1234], dtype=np.uint16)
    return bits.view(np.uint8).copy()


def main() -> None:
    O.build(force=True)
    assert O.have_ref(), "reference sources not found; cannot regenerate fixtures"
    out = {}
    for fmt, name, edge in ((synth.Q8_0, "q8_0", edge_q8_0), (synth.Q4_0, "q4_0", edge_q4_0),
                            (synth.Q4_K, "q4_k", edge_q4_k), (synth.Q5_K, "q5_k", edge_q5_k),
                            (synth.Q6_K, "q6_k", edge_q6_k), (synth.BF16, "bf16", edge_bf16)):
        e = edge()
        be = synth.BLOCK_ELEMS[fmt]
        n_edge = e.size // synth.BLOCK_BYTES[fmt] * be
        out[f"{name}_edge_raw"] = e
        out[f"{name}_edge_f32bits"] = O.ref_dequant(fmt, e, 1, n_edge).view(np.uint32).reshape(-1)
        rows, cols = 6, 768
        r = synth.make_weights(fmt, rows, cols, seed=1000 + fmt)
        out[f"{name}_rand_raw"] = r
        out[f"{name}_rand_shape"] = np.array([rows, cols], dtype=np.int64)
        out[f"{name}_rand_f32bits"] = O.ref_dequant(fmt, r, rows, cols).view(np.uint32).reshape(-1)
        if fmt in (synth.Q8_0, synth.Q4_0):
            vals, scales = O.ref_separate(fmt, r, rows, cols)
            out[f"{name}_rand_sep_values"] = vals.view(np.uint8)
            out[f"{name}_rand_sep_scales"] = scales

    exe = os.path.join("/tmp", "gen_testdata")
    subprocess.run(["g++", "-O2", "-std=c++17", "-o", exe, os.path.join(HERE, "gen_testdata.cpp")], check=True)

    def draw(lo, hi, seed, count):
        raw = subprocess.run([exe, repr(lo), repr(hi), str(seed), str(count)], check=True, capture_output=True).stdout
        return np.frombuffer(raw, dtype=np.float32).copy()

    out["mt19937_42_uniform_0p1_10"] = draw(0.1, 10.0, 42, 1024)
    out["mt19937_42_uniform_m1_1"] = draw(-1.0, 1.0, 42, 4 * 5120)
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", os.path.join(HERE, "golden.npz"), os.path.getsize(os.path.join(HERE, "golden.npz")), "bytes")


if __name__ == "__main__":
    main()
