"""Per-variant timing of the quantized matmul, and tuning rules derived from it.

The reference times every compiled Q4 / Q8 matmul variant on a list of decode and prefill shapes and
writes one JSON record per shape (benchmarks/op_bench.cpp:505-680: `QuantMatMul.raw_data[i] =
{shape, q8: [{variant, name, median_us, gflops}], q8_silu: [...], q4: [...]}`); a separate script turns
such records into `tuning_data.json` rules that `VariantSelector::select` consults
(runtime/VariantSelector.cpp:283-428: `operators.<Op>.backends.<backend>.{default_variant,
rules[{variant, conditions{shape}}]}`, first match wins).

This module does both for the B200 kernels:

    python -m cut_b200.op_bench --out op_bench.json [--rules tuning_data.json]

times the three variants of the block-layout matmul (`MatMulQBlocks`: 0 any-shape SIMT kernel,
1 decode mat-vec, 2 tensor-core GEMM) for Q8_0 / Q4_0 / Q4_K, plain and with the SiLU epilogue, plus
the two plane-layout kernels (`q8`, `q4`: the reference's operands and its own synthetic data), on the
reference's shapes and the benchmark configurations; `--rules` writes a rule for every shape whose
fastest variant is not the built-in choice.  Inputs are generated on the device side of torch
(device memory and streams only); every launch goes through the C ABI.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys

import numpy as np

# (M, K, N): the reference's list (op_bench.cpp:509-518) and the benchmark configurations around it
REFERENCE_SHAPES = [(1, 2048, 2048), (1, 4096, 4096), (1, 4096, 11008), (8, 2048, 2048), (8, 2048, 5632), (32, 2048, 2048),
                    (32, 2048, 5632), (128, 2048, 2048), (128, 2048, 5632), (512, 2048, 2048), (512, 2048, 5632)]
EXTRA_SHAPES = [(8, 4096, 11008), (16, 4096, 11008), (32, 4096, 11008), (1, 4096, 14336), (512, 4096, 14336), (1, 8192, 8192),
                (8, 8192, 8192), (16, 8192, 8192), (32, 8192, 8192), (1, 28672, 8192), (8, 28672, 8192),
                # batch 32 and 64 on the 70B projections and on their row shards over 8 GPUs: where the mat-vec in row groups
                # can beat the GEMM's fixed cost
                (32, 8192, 28672), (32, 28672, 8192), (32, 8192, 1024), (32, 8192, 3584), (32, 28672, 1024), (64, 8192, 1024),
                (32, 4096, 4096), (24, 4096, 11008)]
BLOCK_VARIANT_NAMES = {0: "QMatMulGeneric", 1: "QGemvBulkMma", 2: "QGemmTcgen05"}
PLANE_VARIANT_NAMES = {0: "QMatMulGeneric", 3: "QGemvPlanes"}
OPERATOR = "MatMulQBlocks"
UNARY_SILU = 133


def builtin_block_variant(M: int, K: int, N: int, a_is_f32: bool) -> int:
    """The choice MatMulOpNode makes without tuning data for raw GGUF blocks."""
    vrows = 2 * M if a_is_f32 else M
    if K % 256 == 0 and vrows <= 16:
        if not a_is_f32 and M >= 13 and K * N >= 1 << 24:
            return 2  # the mat-vec's fourth column tile loses to the GEMM for few tokens on 16 M weights and more
        return 1
    if K % 256 == 0 and M > 1:
        return 2
    return 0


def derive_rules(records: list[dict], key: str = "blocks_q4_0", min_gain: float = 0.10) -> dict:
    """tuning_data.json content from op_bench records: one exact-shape rule for every shape whose fastest
    variant under `key` differs from the built-in choice (fp16 activations, as the records are timed) and beats it
    by at least `min_gain` (a rule is not worth a run-to-run wobble)."""
    rules = []
    for rec in records:
        rows = rec.get(key) or []
        if not rows:
            continue
        best = min(rows, key=lambda r: r["median_us"])
        M, K, N = rec["shape"]
        builtin = builtin_block_variant(M, K, N, False)
        if best["variant"] != builtin:
            base = next((r["median_us"] for r in rows if r["variant"] == builtin), None)
            if base is not None and best["median_us"] > (1.0 - min_gain) * base:
                continue
            was = f" (built-in {BLOCK_VARIANT_NAMES[builtin]} {base:.2f} us)" if base is not None else ""
            rules.append({"variant": best["variant"], "conditions": {"shape": [M, K, N]},
                          "comment": f"{best['name']} {best['median_us']:.2f} us{was}"})
    # default_variant -1: shapes without a rule keep the operator's built-in choice (it depends on the shape)
    return {"operators": {OPERATOR: {"backends": {"cuda": {"default_variant": -1, "rules": rules}}}}}


def _time_graph(torch, launch_all, launches: int, rounds: int = 5) -> float:
    """Median over `rounds` of the device time per launch of a CUDA-graph chain."""
    launch_all()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        launch_all()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    iters = max(2, 400 // launches)
    samples = []
    for _ in range(rounds):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        samples.append(a.elapsed_time(b) * 1e3 / (iters * launches))
    del g
    return statistics.median(samples)


def time_blocks(torch, dev, fmt: int, M: int, K: int, N: int, variant: int, silu: bool) -> float | None:
    """Median us of one block-layout matmul forced to `variant` (weights cycled past L2), or None if the
    variant does not take the shape."""
    from . import _lib as L
    from . import ops, synth

    rb = synth.row_bytes(fmt, K)
    reps = max(2, min(32, int(300e6 // (N * rb)) + 1))
    base = torch.from_numpy(synth.make_weights(fmt, N, K, seed=17)).to(dev)
    W = torch.empty((reps, base.numel()), dtype=torch.uint8, device=dev)
    for r in range(reps):
        W[r] = torch.roll(base, shifts=synth.BLOCK_BYTES[fmt] * 7 * r)
    A = torch.from_numpy(synth.make_activations(M, K, 18, np.float16)).to(dev)
    C = torch.zeros((M, N), dtype=torch.float32, device=dev)
    descs, ws = [], None
    for r in range(reps):
        d, _, _ = ops.make_desc(A, W[r], fmt, N, C_out=C, variant=variant,
                                fusion_type=L.FUSION_UNARY if silu else L.FUSION_NONE, fusion_op=UNARY_SILU if silu else 0)
        need = ops.workspace_bytes(d)
        if need:
            ws = ws if ws is not None else torch.empty(need, dtype=torch.uint8, device=dev)
            d.workspace, d.workspace_bytes = ws.data_ptr(), need
        descs.append(d)
    try:
        ops.launch(descs[0])
    except L.CutbError:
        return None

    def launch_all():
        for d in descs:
            ops.launch(d)

    return _time_graph(torch, launch_all, reps)


def time_planes(torch, dev, q4: bool, M: int, K: int, N: int, silu: bool, variant: int) -> float | None:
    """Median us of the plane-layout matmul forced to `variant` (0 any-shape kernel, 3 coalesced mat-vec) on the
    reference's own synthetic operands (op_bench.cpp:527-537; one weight tensor, as there), or None if the
    variant does not take the shape."""
    from . import _lib as L
    from . import ops

    i = np.arange(K * (N // 2 if q4 else N), dtype=np.int64)
    if q4:
        B = (((i * 5 + 1) % 16) | (((i * 3 + 2) % 16) << 4)).astype(np.uint8).reshape(K, N // 2)
    else:
        B = ((i * 7 + 3) % 21 - 10).astype(np.int8).view(np.uint8).reshape(K, N)
    S = np.full((K // 32, N), 0x3C00, dtype=np.uint16)
    A = torch.from_numpy(np.random.default_rng(42).standard_normal((M, K)).astype(np.float32)).to(dev)
    Bd, Sd = torch.from_numpy(B).to(dev), torch.from_numpy(S).to(dev)
    C = torch.zeros((M, N), dtype=torch.float32, device=dev)
    d, _, _ = ops.make_desc(A, Bd, L.Q4_0 if q4 else L.Q8_0, N, layout=L.LAYOUT_KN_PLANES, scales=Sd, ldb=Bd.stride(0), lds=N, C_out=C,
                            variant=variant, fusion_type=L.FUSION_UNARY if silu else L.FUSION_NONE, fusion_op=UNARY_SILU if silu else 0)
    need = ops.workspace_bytes(d)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    try:
        ops.launch(d)
    except L.CutbError:
        return None
    return _time_graph(torch, lambda: ops.launch(d), 1)


def run(shapes, planes_limit: float = 2.5e8) -> list[dict]:
    import torch

    from . import _lib as L

    if not torch.cuda.is_available():
        raise SystemExit("op_bench needs a CUDA device")
    dev = torch.device("cuda", torch.cuda.current_device())
    L.lib()
    records = []
    for M, K, N in shapes:
        rec = {"shape": [M, K, N]}
        flops = 2.0 * M * K * N
        for key, fmt in (("blocks_q8_0", L.Q8_0), ("blocks_q4_0", L.Q4_0), ("blocks_q4_k", L.Q4_K)):
            for silu in (False, True):
                rows = []
                for v in (0, 1, 2):
                    if v == 0 and flops > planes_limit * 40:  # the any-shape kernel on prefill shapes takes seconds
                        continue
                    us = time_blocks(torch, dev, fmt, M, K, N, v, silu)
                    if us is not None:
                        rows.append({"variant": v, "name": BLOCK_VARIANT_NAMES[v], "median_us": round(us, 4),
                                     "gflops": round(flops / (us * 1e3), 2)})
                rec[key + ("_silu" if silu else "")] = rows
        if flops <= planes_limit:
            for key, q4, silu in (("q8", False, False), ("q8_silu", False, True), ("q4", True, False)):
                rows = []
                for v in (0, 3):
                    us = time_planes(torch, dev, q4, M, K, N, silu, v)
                    if us is not None:
                        rows.append({"variant": v, "name": PLANE_VARIANT_NAMES[v], "median_us": round(us, 4),
                                     "gflops": round(flops / (us * 1e3), 2)})
                rec[key] = rows
        print(f"QuantMatMul M={M} K={K} N={N} done", file=sys.stderr, flush=True)
        records.append(rec)
        torch.cuda.empty_cache()
    return records


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", default="-", help="where the op_bench JSON goes (default: stdout)")
    ap.add_argument("--rules", default=None, help="also write tuning_data.json rules derived from the run")
    ap.add_argument("--reference-shapes-only", action="store_true")
    ap.add_argument("--only", nargs=3, type=int, metavar=("M", "K", "N"),
                    help="time one shape only and print its record (a small, fixed workload for a profiler)")
    ap.add_argument("--format", choices=["q8_0", "q4_0", "q4_k"], default="q4_0", help="with --only: block format")
    ap.add_argument("--layout", choices=["blocks", "planes"], default="blocks", help="with --only: weight layout")
    ap.add_argument("--variant", type=int, default=None, help="with --only: force this variant (default: the built-in choice)")
    ap.add_argument("--silu", action="store_true", help="with --only: fuse SiLU into the epilogue (the *_silu records)")
    args = ap.parse_args(argv)
    import torch

    if args.only:
        from . import _lib as L

        if not torch.cuda.is_available():
            raise SystemExit("op_bench needs a CUDA device")
        dev = torch.device("cuda", torch.cuda.current_device())
        M, K, N = args.only
        if args.layout == "planes":
            v = 3 if args.variant is None else args.variant
            us = time_planes(torch, dev, args.format != "q8_0", M, K, N, args.silu, v)
        else:
            fmt = {"q8_0": L.Q8_0, "q4_0": L.Q4_0, "q4_k": L.Q4_K}[args.format]
            v = builtin_block_variant(M, K, N, False) if args.variant is None else args.variant
            us = time_blocks(torch, dev, fmt, M, K, N, v, args.silu)
        print(json.dumps({"shape": [M, K, N], "format": args.format, "layout": args.layout, "variant": v, "silu": args.silu, "median_us": us}))
        return 0

    shapes = REFERENCE_SHAPES if args.reference_shapes_only else REFERENCE_SHAPES + EXTRA_SHAPES
    records = run(shapes)
    doc = {"device": torch.cuda.get_device_name(), "operators": {"QuantMatMul": {"raw_data": records}}}
    text = json.dumps(doc, indent=1)
    if args.out == "-":
        print(text)
    else:
        with open(args.out, "w") as f:
            f.write(text + "\n")
    if args.rules:
        with open(args.rules, "w") as f:
            f.write(json.dumps(derive_rules(records), indent=1) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
