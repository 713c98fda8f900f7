"""Regenerates the golden fixtures in this directory.

Run from the repository root in a container that has the reference checked out
(the fixtures themselves are committed, so the tests never need it):

    python tests/golden/make_golden.py

It (1) builds oracle/_ref/libcutref.so from the reference's unmodified
gguf_reader.cpp, (2) pushes hand-crafted edge-case blocks and seeded random
blocks of Q8_0 / Q4_0 / Q4_K (and Q5_K / Q6_K / BF16, which only the dequant
operator takes) through the reference's GGUFReader and stores the
raw bytes next to the float32 bit patterns and separated planes it returned,
(3) stores the mt19937 activation vectors of the reference's own tests, and
(4) builds oracle/_ref/libcutref_runner.so (the reference runner's translation
unit, reached through oracle/ref_runner_shim.cpp) and stores what its file-static
re-encoders return: float -> half conversions of edge values, Q8_0 quantisation of
seeded rows, and the affine re-encode of Q4_K tensors.
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


def edge_q4_1() -> np.ndarray:
    mins = [0x0000, 0x8000, 0x0001, 0x3C00, 0xBC00, 0x7BFF, 0xFBFF, 0x2E66, 0x83FF, 0x0400, 0x1234, 0xB266]
    blocks = np.zeros((len(EDGE_D) * 2, 20), dtype=np.uint8)
    for i, d in enumerate(EDGE_D):
        for v in range(2):
            b = blocks[2 * i + v]
            b[0:2] = np.array([d], dtype=np.uint16).view(np.uint8)
            b[2:4] = np.array([mins[(i + 5 * v) % len(mins)]], dtype=np.uint16).view(np.uint8)
            nib = (np.arange(32) % 16) if v == 0 else np.array([0, 15, 8, 7] * 8)
            b[4:] = (nib[:16] | (nib[16:] << 4)).astype(np.uint8)
    return blocks.reshape(-1)


def edge_q5_0() -> np.ndarray:
    blocks = np.zeros((len(EDGE_D) * 2, 22), dtype=np.uint8)
    for i, d in enumerate(EDGE_D):
        for v in range(2):
            b = blocks[2 * i + v]
            b[0:2] = np.array([d], dtype=np.uint16).view(np.uint8)
            qh = 0xA5C3F00F if v == 0 else (0xFFFFFFFF if i % 2 else 0x00000001 << (i % 32))
            b[2:6] = np.array([qh], dtype=np.uint32).view(np.uint8)
            nib = (np.arange(32) % 16) if v == 0 else np.array([0, 15, 8, 7] * 8)
            b[6:] = (nib[:16] | (nib[16:] << 4)).astype(np.uint8)
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
                            (synth.Q6_K, "q6_k", edge_q6_k), (synth.BF16, "bf16", edge_bf16),
                            (synth.Q4_1, "q4_1", edge_q4_1), (synth.Q5_0, "q5_0", edge_q5_0)):
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

    # (4) the runner's re-encoders (interface/runner/llama/llama.cpp:445-619), run from the reference's own source
    assert O.have_ref_runner(), "the runner shim was not built; cannot regenerate its fixtures"
    rr = O.ref_runner()
    edge_f32 = np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65519.9, 65520.0, 1e5, -1e5, 6.1035156e-05, 6.0975552e-05, 5.9604645e-08,
                         2.9802322e-08, 2.9802326e-08, 1e-8, 0.1, 0.33333334, 1.0009766, 1.0004883, 1.0014648, 2047.5, 2048.5,
                         np.inf, -np.inf, 3.1415927, 1e-5, 7.5e-5, 0.00012207031], dtype=np.float32)
    rng = np.random.default_rng(4242)
    rand_f32 = np.concatenate([edge_f32, (rng.standard_normal(2000) * np.exp(rng.uniform(-18, 11, 2000))).astype(np.float32)])
    out["runner_f32_in"] = rand_f32
    out["runner_f32_to_f16"] = np.array([rr.cutref_runner_f32_to_f16(float(v)) for v in rand_f32], dtype=np.uint16)
    halves = np.concatenate([np.array(EDGE_D + [0x7C00, 0xFC00, 0x7E00], dtype=np.uint16), rng.integers(0, 65536, 1000).astype(np.uint16)])
    out["runner_f16_in"] = halves
    out["runner_f16_to_f32_bits"] = np.array([rr.cutref_runner_f16_to_f32(int(h)) for h in halves], dtype=np.float32).view(np.uint32)
    x = (rng.standard_normal(64 * 32) * np.repeat(np.exp(rng.uniform(-12, 6, 64)), 32)).astype(np.float32)
    x[:32] = 0.0                       # an all-zero block: d = 0, id = 0
    x[32:64] = np.linspace(-1, 1, 32)  # ties of lroundf at +-0.5 steps of d
    x[64:96] = 127.0
    qv, qs = O.ref_runner_quantize_rows_q8_0(x)
    out["runner_q8_in"], out["runner_q8_values"], out["runner_q8_scales"] = x, qv.view(np.uint8), qs
    for tag, (n, k, seed) in {"a": (8, 512, 77), "b": (34, 256, 78)}.items():
        rawk = synth.make_weights(synth.Q4_K, n, k, seed=seed)
        if tag == "b":  # the edge-case super-blocks of the dequant fixtures in front (subnormal d / dmin, 6-bit extremes)
            e = edge_q4_k()
            rawk[: e.size] = e
        pt, st = O.ref_runner_requant_q4k_affine(rawk, n, k)
        out[f"runner_requant_{tag}_raw"], out[f"runner_requant_{tag}_shape"] = rawk, np.array([n, k], dtype=np.int64)
        out[f"runner_requant_{tag}_packed"], out[f"runner_requant_{tag}_scales"] = pt, st

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
