#!/usr/bin/env python
"""Benchmark of the GGUF quantized-matmul decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the Q4_0 decode mat-vec at the 7B FFN shape -- weight
11008 x 4096 stored as GGUF Q4_0 blocks, fp16 activation, batch 1 (the second
benchmark configuration).  One step = one pass over REPLICAS distinct weight
tensors (a 32-layer stack's worth, 811 MB), one kernel launch per tensor,
replayed from a CUDA graph; cycling distinct tensors keeps the 25 MB weights
from being served by the 126 MB L2.  The metric is algorithmic bytes (weights
+ activations + output, each counted once) per second, in GB/s.

N > 1: every rank holds its own 11008-row shard of a [N x 11008, 4096] weight
(row sharding: weights never move), computes its output slice and an NCCL
all-gather assembles the full output on every rank once per step ("weak"
scaling: per-GPU work is fixed).

Besides the device-resident number (`value`) the line carries `e2e` (same
metric through the host-buffer calls: every step uploads its activations from
pinned host memory, runs its mat-vecs and downloads their results), `roofline` (achieved GB/s of the mat-vec
kernel against the measured HBM copy peak), `cpu_baseline` (the CPU checker
timed on this host) and the SM clocks sampled during the timed region.

`--impl reference` times the reference's own CPU implementation of the path
instead (its GGUF reader's dequantiser + the scalar contraction of its test
harness) on a bounded sample and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

FMT_NAME = "Q4_0"
N_ROWS, K_COLS, BATCH = 11008, 4096, 1
REPLICAS = 32
METRIC = "qgemv_hbm_gbs"
UNIT = "GB/s"
WORKLOAD = f"configs[1]: {FMT_NAME} decode mat-vec {N_ROWS}x{K_COLS} (GGUF blocks), fp16 activation, batch {BATCH}"

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one mat-vec launch of this workload, from an ncu
# capture of this kernel (a profiler cannot run inside the timed region, so the figure is carried here and the
# line says where it comes from).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 25_419_520


def algorithmic_bytes(n_rows: int, k: int, batch: int) -> int:
    """Weights once + fp16 activations + fp32 output (what the roofline counts)."""
    return n_rows * (k // 32) * 18 + batch * k * 2 + batch * n_rows * 4


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Polls SM clock, power and throttle reasons through NVML while the timed
    region runs (read-only queries)."""

    def __init__(self, index: int, period_s: float = 0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=1.0)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
            "power_w_max": max(self.power) if self.power else None,
        }


def cpu_port_throughput(budget_s: float):
    """The CPU checker's mat-vec (all host threads) on the same workload, bounded
    to about `budget_s` seconds; returns (GB/s, threads, description)."""
    from cut_b200 import synth
    from oracle import oracle as O

    n_rep = 4
    ws = [synth.make_weights(synth.Q4_0, N_ROWS, K_COLS, seed=9000 + i) for i in range(n_rep)]
    a = synth.make_activations(BATCH, K_COLS, 77, np.float16).astype(np.float32)
    O.qmatmul_blocks_fast(synth.Q4_0, a, ws[0], BATCH, K_COLS, N_ROWS)
    t0 = time.perf_counter()
    calls = 0
    while time.perf_counter() - t0 < budget_s:
        O.qmatmul_blocks_fast(synth.Q4_0, a, ws[calls % n_rep], BATCH, K_COLS, N_ROWS)
        calls += 1
    dt = time.perf_counter() - t0
    gbs = calls * algorithmic_bytes(N_ROWS, K_COLS, BATCH) / dt / 1e9
    return gbs, O.num_threads(), f"{calls} mat-vecs of {N_ROWS}x{K_COLS} {FMT_NAME} over {n_rep} weight copies in {dt:.1f} s"


def run_reference(args) -> None:
    """Reference arm: the reference's CPU code for the path on this host's cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from cut_b200 import synth
    from oracle import oracle as O

    sample_rows = N_ROWS  # one step = one whole mat-vec of the workload (about 0.15 s on this path)
    w = synth.make_weights(synth.Q4_0, sample_rows, K_COLS, seed=9100)
    a = synth.make_activations(BATCH, K_COLS, 77, np.float16).astype(np.float32)
    use_ref = O.have_ref()
    path = O.ref_write_file(synth.Q4_0, w, sample_rows, K_COLS) if use_ref else None

    def one_step():
        if use_ref:
            # the reference's own reader + dequantiser (single-threaded, as it runs)
            wf = O.ref_dequant_path(path, sample_rows, K_COLS)
        else:
            wf = O.dequant_rows(synth.Q4_0, w, sample_rows, K_COLS)
        # scalar float contraction of the reference's test harness, rows spread over all threads
        return O.matmul_dense(a, wf)

    for _ in range(args.warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_step()
    dt = time.perf_counter() - t0
    if path:
        os.unlink(path)
    bytes_per_step = algorithmic_bytes(sample_rows, K_COLS, BATCH)
    val = args.steps * bytes_per_step / dt / 1e9
    kind = "reference" if use_ref else "port"
    sample = (f"{args.steps} steps of one {sample_rows}x{K_COLS} {FMT_NAME} mat-vec (the whole workload tensor): "
              + ("dequantised by the reference's gguf_reader.cpp (1 thread), " if use_ref else "dequantised by the C port, ")
              + "contracted by the restated scalar loop of its test harness (all threads)")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "host": "cpu"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": O.num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    try:
        ref_gpu = reference_cuda_measurement()
    except Exception as e:  # noqa: BLE001  (context only: the arm's number is the CPU one)
        ref_gpu = {"error": f"{type(e).__name__}: {e}"}
    if ref_gpu:
        line["config"]["also_measured"] = {"reference_cuda_kernels_on_this_gpu": ref_gpu}
    print(json.dumps(line), flush=True)


def reference_cuda_measurement() -> dict | None:
    """The reference's OWN CUDA kernels on this GPU, as context for the reference arm (its decode path when its CUDA
    backend runs: MatMulQ4GemvKPar8 / MatMulQ8GemvKPar8 over the [K, N] plane layout, compiled by NVRTC from the
    reference tree into oracle/_ref/cuda by oracle/build_ref_cuda.py).  Same workloads as the GPU arm: configs[1]
    (Q4_0 11008 x 4096, batch 1; the reference's kernels take fp32 activations) and configs[0] (Q8_0 4096 x 4096),
    weights cycled over distinct copies so that L2 cannot serve them, one CUDA graph per pass.  None without a GPU or
    without the cubins."""
    try:
        import torch

        from oracle import ref_cuda
    except Exception:  # noqa: BLE001
        return None
    if not torch.cuda.is_available() or not ref_cuda.have("MatMulQ4GemvKPar8"):
        return None
    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    out = {}
    for key, kernel, fmt, n, k in (("configs[1]_q4_0_11008x4096_batch1", "MatMulQ4GemvKPar8", L.Q4_0, N_ROWS, K_COLS),
                                   ("configs[0]_q8_0_4096x4096_batch1", "MatMulQ8GemvKPar8", L.Q8_0, 4096, 4096)):
        if not ref_cuda.have(kernel):
            continue
        q4 = fmt == L.Q4_0
        raw = torch.from_numpy(synth.make_weights(fmt, n, k, seed=71)).to(dev)
        vals, scales = ops.separate_blocks(raw, fmt, n, k)
        plane = ops.transpose_q4(vals, n, k) if q4 else ops.transpose_2d(vals, ldo=(n + 3) // 4 * 4)
        scalesT = ops.transpose_2d(scales, ldo=(n + 3) // 4 * 4)
        reps = max(2, int(600e6 // plane.numel()) + 1)
        P = torch.stack([torch.roll(plane, shifts=13 * r, dims=1) for r in range(reps)])
        A = torch.from_numpy(synth.make_activations(1, k, 72, np.float32)).to(dev)
        C = torch.zeros((reps, 1, n), dtype=torch.float32, device=dev)

        def sweep():
            for r in range(reps):
                ref_cuda.launch(kernel, A, P[r], scalesT, C[r], 1, k, n, stride_a=k, stride_b=plane.stride(0), stride_c=n,
                                scale_stride=scalesT.stride(0))

        sweep()
        torch.cuda.synchronize()
        want = ops.qmatmul(A, raw, fmt, n)  # replica 0 is not rotated: the block kernel on the same weights
        rel = float(torch.linalg.norm(C[0] - want) / torch.linalg.norm(want))
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            sweep()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = 10
        a.record()
        for _ in range(iters):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / (iters * reps)
        nbytes = plane.numel() + scalesT.numel() * 2 + k * 4 + n * 4
        out[key] = {"kernel": kernel, "us_per_launch": us, "GB/s": nbytes / us / 1e3, "algorithmic_bytes": nbytes,
                    "weight_copies": reps, "rel_l2_vs_block_kernel": rel}
        del g, P, C
        torch.cuda.empty_cache()
    # prefill: its tensor-core tiled kernel on the configs[2] shape (Q4_0 planes; the GPU arm's GEMM reads Q4_K blocks
    # of the same shape, and Q4_0 blocks in 60 us)
    if ref_cuda.have("MatMulQ4CoopMatTiled"):
        m, k, n = 512, 4096, 14336
        raw = torch.from_numpy(synth.make_weights(L.Q4_0, n, k, seed=73)).to(dev)
        vals, scales = ops.separate_blocks(raw, L.Q4_0, n, k)
        plane, scalesT = ops.transpose_q4(vals, n, k), ops.transpose_2d(scales, ldo=n)
        A = torch.from_numpy(synth.make_activations(m, k, 74, np.float32)).to(dev)
        C = torch.zeros((m, n), dtype=torch.float32, device=dev)
        run = lambda: ref_cuda.launch("MatMulQ4CoopMatTiled", A, plane, scalesT, C, m, k, n, stride_a=k, stride_b=plane.stride(0),
                                      stride_c=n, scale_stride=n)
        for _ in range(2):
            run()
        torch.cuda.synchronize()
        want = ops.qmatmul(A, raw, L.Q4_0, n)
        rel = float(torch.linalg.norm(C - want) / torch.linalg.norm(want))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            run()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / 5
        out["configs[2]_shape_q4_0_512x4096x14336"] = {"kernel": "MatMulQ4CoopMatTiled", "us_per_launch": us,
                                                       "TFLOP/s": 2.0 * m * k * n / us / 1e6, "rel_l2_vs_block_gemm": rel}
    # decode attention at the configs[3] geometry (32 query / 8 KV heads of 128, fp16 cache, 515 populated rows)
    if ref_cuda.have("Attention_f16"):
        nh, nkv, hd, rows, seq = 32, 8, 128, 2048, 515
        gen = torch.Generator(device=dev).manual_seed(7)
        q = torch.randn(nh * hd, generator=gen, device=dev)
        kc = torch.randn((rows, nkv * hd), generator=gen, device=dev).half()
        vc = torch.randn((rows, nkv * hd), generator=gen, device=dev).half()
        params = torch.tensor([seq - 1, seq], dtype=torch.int32, device=dev)
        o_ref = torch.zeros(nh * hd, device=dev)
        ws = ops.attention_workspace(nh, nkv, hd, rows, dev)
        scale = 1.0 / float(np.sqrt(np.float32(hd)))

        def time_us(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(50):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) * 1e3 / 50

        us_ref = time_us(lambda: ref_cuda.attention(True, q, kc, vc, params, o_ref, nh, nkv, hd, scale))
        o_own = ops.attention_decode(q, kc, vc, params, nh, nkv, hd, ws, scale=scale)
        us_own = time_us(lambda: ops.attention_decode(q, kc, vc, params, nh, nkv, hd, ws, out=o_own, scale=scale))
        out["configs[3]_decode_attention_515_rows"] = {"kernel": "Attention (Float16 cache)", "us_per_launch": us_ref,
                                                       "this_library_us_per_launch": us_own,
                                                       "max_abs_diff": float((o_own - o_ref).abs().max())}
    # prefill attention at the same geometry: a 512-token prompt over an empty cache (the reference serves one token
    # and query head per block; this library 64 tokens of a head per block on the tensor cores)
    if ref_cuda.have("BatchedAttentionReadCache_f16"):
        nh, nkv, hd, rows, T = 32, 8, 128, 1024, 512
        gen = torch.Generator(device=dev).manual_seed(8)
        q = torch.randn((T, nh * hd), generator=gen, device=dev)
        kc = torch.randn((rows, nkv * hd), generator=gen, device=dev).half()
        vc = torch.randn((rows, nkv * hd), generator=gen, device=dev).half()
        ang = torch.rand((rows, hd // 2), generator=gen, device=dev) * 6.28
        cos_t, sin_t = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
        pos = torch.arange(0, T, dtype=torch.int32, device=dev)
        scale = 1.0 / float(np.sqrt(np.float32(hd)))
        o_ref = torch.zeros((T, nh * hd), device=dev)

        def time_us2(fn, n=20):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) * 1e3 / n

        us_ref = time_us2(lambda: ref_cuda.batched_attention(True, q, kc, vc, pos, cos_t, sin_t, o_ref, T, nh, nkv, hd, scale, nh * hd, 0))
        o_own = ops.batched_attention(q, kc, vc, pos, cos_t, sin_t, nh, nkv, hd)
        us_own = time_us2(lambda: ops.batched_attention(q, kc, vc, pos, cos_t, sin_t, nh, nkv, hd, out=o_own))
        out["configs[3]_prefill_attention_512_tokens"] = {
            "kernel": "BatchedAttentionReadCache (Float16 cache)", "us_per_launch": us_ref, "this_library_us_per_launch": us_own,
            "max_abs_diff": float((o_own - o_ref).abs().max()),
            "note": "this library rounds rotated queries and probabilities to fp16 for the tensor cores; sums are fp32"}
    return out or None


def decode_measurement(dev, n_layers: int = 32, steps: int = 256, graph: bool = True, synthetic_cache: bool = False,
                       weights: dict | None = None) -> dict:
    """configs[3]: Llama-style decoder (hidden 4096, 32 query / 8 KV heads of 128, FFN 14336, vocab 32000, Q4_K
    projections, fp16 KV cache of 2048 rows): a prompt of 512 random token ids, then batch-1 greedy decode of
    `steps` tokens.  The prompt runs as one batch (tensor-core GEMM projections, batched RoPE cache write, one
    attention block per KV head and token; timed separately as prefill_ms, not part of tok/s), so every decode
    step attends over the 512 + t rows the model itself wrote.  Layer 0's weights are generated, the other layers are row
    rotations of them at their own addresses (4 GB in all)."""
    import torch

    from cut_b200.llama_decode import LlamaConfig, LlamaDecoder, synthetic_weights

    cfg = LlamaConfig(n_layers=n_layers)
    # super-block scales divided by 128: the configuration's Q4_K distribution has a positive mean (~2), every
    # projection then sums coherently and SiLU(gate) * up leaves fp16, the operand type of the prefill GEMM
    dec = LlamaDecoder(cfg, weights if weights is not None else synthetic_weights(cfg, seed=41, distinct_layers=False, scale_shift=7), dev)
    prompt = np.random.default_rng(42).integers(0, cfg.vocab, 512)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    if synthetic_cache:  # profiling aid: no prompt run, cache rows 0..511 ~N(0, 1), one step at position 512
        gen = torch.Generator(device=dev).manual_seed(42)
        for l in range(cfg.n_layers):
            dec.k_cache[l][:512].copy_(torch.randn((512, cfg.kv_dim), generator=gen, device=dev))
            dec.v_cache[l][:512].copy_(torch.randn((512, cfg.kv_dim), generator=gen, device=dev))
        logits = dec.step(int(prompt[-1]), 512)
    else:
        dec.prefill(prompt)  # warm-up of the batch path (first-use kernel attributes, allocator)
        torch.cuda.synchronize()
        p0.record()
        logits = dec.prefill(prompt)
    p1.record()
    torch.cuda.synchronize()
    prompt_ms = p0.elapsed_time(p1)
    finite = bool(torch.isfinite(logits).all())
    first = int(torch.argmax(logits).item())
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        dec.set_position(first, 512)
        dec.capture()
        dec.replay(3)
        dec.set_position(first, 512)
        torch.cuda.synchronize()
        a.record()
        dec.replay(steps)
        b.record()
    else:  # eager: one launch per call, for a profiler's launch list
        tok = first
        torch.cuda.synchronize()
        a.record()
        for t in range(steps):
            dec.step(tok, 512 + t)
        b.record()
    torch.cuda.synchronize()
    dec.check_status()
    ms = a.elapsed_time(b)
    wb = dec.weight_bytes_per_token()
    return {"tok/s": steps * 1e3 / ms, "ms_per_token": ms / steps, "tokens": steps, "layers": cfg.n_layers,
            "weight_bytes_per_token": wb, "weight_GB/s": wb * steps / ms / 1e6, "kernel_launches_per_token": dec.launches_per_step,
            "logits_finite": finite, "graph": graph,
            "kv_cache": "fp16; rows 0..511 synthetic" if synthetic_cache else
            "fp16; rows 0..511 written by the batched prefill of the 512-token prompt",
            "prefill_ms": prompt_ms, "prefill_tok/s": 512e3 / prompt_ms,
            "activations": "fp32, staged at 16 bits per 32-k block"}


def cpp_runner_measurement(device_index: int, cfg, weights: dict, steps: int = 128) -> dict:
    """configs[3] through the C++ host: the same synthetic model written as a GGUF file, loaded by GGUFFile / GGUFUploader
    (fused QKV, paired gate / up rows), the per-token step recorded by LlamaRunner over the operator API into one
    reusable command buffer and replayed per token.  Per token the host writes {pos, seqLen} and the token id, resubmits,
    waits and reads the arg-max back, as the reference's runner does (interface/runner/llama/llama.cpp:2090-2166), so
    tok/s here includes that round trip.  A 16-token prompt is fed token by token, then `steps` greedy tokens are timed."""
    import tempfile

    from cut_b200.llama_decode import run_cpp_runner, write_model_gguf

    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "model.gguf")
        write_model_gguf(path, cfg, weights)
        prompt = np.random.default_rng(42).integers(0, cfg.vocab, 16)
        r = run_cpp_runner(path, prompt, steps, device=device_index, max_seq=cfg.max_seq)
    return {"tok/s": steps / r["seconds"], "ms_per_token": 1e3 * r["seconds"] / steps, "tokens": steps,
            "dispatches_per_token": r["dispatches_per_token"], "weight_bytes_per_token": r["weight_bytes_per_token"],
            "weight_GB/s": r["weight_bytes_per_token"] * steps / r["seconds"] / 1e9,
            "host_round_trip_per_token": True, "context": "positions 16..%d" % (16 + steps - 1),
            "path": "GGUF file -> GGUFUploader -> LlamaRunner (Operations, reusable command buffer) in libcut_host.so"}


def chain_us(dev, fmt: int, n: int, k: int, m: int, act_dtype, flags: int = 0, total_mb: float = 600.0, seed: int = 51) -> dict:
    """Device time of one quantized matmul over GGUF blocks inside a CUDA-graph chain of launches that cycle
    through enough distinct weight tensors (>= total_mb, so L2 cannot serve them); returns us per launch, the
    algorithmic GB/s (weights + activations + output once each) and the variant that ran."""
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    rb = synth.row_bytes(fmt, k)
    reps = max(2, min(64, int(total_mb * 1e6 // (n * rb)) + 1))
    base = torch.from_numpy(synth.make_weights(fmt, n, k, seed=seed)).to(dev)
    W = torch.empty((reps, base.numel()), dtype=torch.uint8, device=dev)
    for r in range(reps):
        W[r] = torch.roll(base, shifts=synth.BLOCK_BYTES[fmt] * 7 * r)
    A = torch.from_numpy(synth.make_activations(m, k, seed + 1, act_dtype)).to(dev)
    C = torch.zeros((reps, m, n), dtype=torch.float32, device=dev)
    descs, keep = [], []
    for r in range(reps):
        d, _, kp = ops.make_desc(A, W[r], fmt, n, C_out=C[r], flags=flags)
        need = ops.workspace_bytes(d)
        if need:
            ws = torch.empty(need, dtype=torch.uint8, device=dev)
            d.workspace, d.workspace_bytes = ws.data_ptr(), need
            kp = kp + (ws,)
        descs.append(d)
        keep.append(kp)
    variant = ops.select_variant(descs[0])

    def sweep():
        for d in descs:
            ops.launch(d)

    sweep()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sweep()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    iters = max(3, int(2000 // reps))
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) * 1e3 / (iters * reps))
    nbytes = n * rb + m * k * A.element_size() + m * n * 4
    del g, W, C
    return {"us_per_launch": best, "GB/s": nbytes / best / 1e3, "algorithmic_bytes": nbytes, "weight_copies": reps,
            "variant": L.lib().cutb_variant_name(variant).decode()}


def planes_chain_us(dev, n: int, k: int) -> dict:
    """Q4_0 mat-vec over the reference's runtime layout ([K, N / 2] nibbles with even n in the low nibble, fp16 scales
    [K / 32, N]: what its loader's plane separation, its Q4 transpose and its scale transpose produce), batch 1,
    weights cycled over distinct copies, in a CUDA graph."""
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    reps = 24
    raw = torch.from_numpy(synth.make_weights(synth.Q4_0, n, k, seed=71)).to(dev)
    vals, scales = ops.separate_blocks(raw, L.Q4_0, n, k)      # [N, K / 2] GGML nibbles, [N, K / 32] f16 bits
    packed = ops.transpose_q4(vals, n, k)                      # [K, pad4(N / 2)]
    scalesT = ops.transpose_2d(scales, ldo=(n + 3) // 4 * 4)   # [K / 32, pad4(N)]
    P = torch.stack([torch.roll(packed, shifts=13 * r, dims=1) for r in range(reps)])
    S = torch.stack([scalesT for _ in range(reps)])
    A = torch.from_numpy(synth.make_activations(1, k, 72, np.float32)).to(dev)
    C = torch.zeros((reps, 1, n), dtype=torch.float32, device=dev)
    descs = [ops.make_desc(A, P[r], L.Q4_0, n, layout=L.LAYOUT_KN_PLANES, scales=S[r], ldb=packed.stride(0), lds=scalesT.stride(0),
                           C_out=C[r]) for r in range(reps)]
    need = ops.workspace_bytes(descs[0][0])
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)  # K-split partial sums; launches are stream-ordered
    for d, _, _ in descs:
        d.workspace, d.workspace_bytes = ws.data_ptr(), need

    def sweep():
        for d, _, _ in descs:
            ops.launch(d)

    sweep()
    torch.cuda.synchronize()
    # the plane kernel against the block kernel on the same weights (replica 0 is not rotated)
    ref = ops.qmatmul(A, raw, L.Q4_0, n)
    rel = float(torch.linalg.norm(C[0] - ref) / torch.linalg.norm(ref))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sweep()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 30
    a.record()
    for _ in range(iters):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) * 1e3 / (iters * reps)
    nbytes = k * (n // 2) + (k // 32) * n * 2 + k * 4 + n * 4
    variant = L.lib().cutb_variant_name(ops.select_variant(descs[0][0])).decode()
    return {"us_per_launch": us, "GB/s": nbytes / us / 1e3, "algorithmic_bytes": nbytes, "variant": variant,
            "rel_l2_vs_block_kernel": rel, "weight_copies": reps}


def planes_gemm_us(dev, m: int, k: int, n: int) -> dict:
    """Prefill over the reference's [K, N] planes (Q4_0 nibbles + fp16 scales, as its unchanged loader and Q4 transpose
    produce them): the tcgen05 GEMM with plane converters, checked against the same GEMM over the GGUF blocks the planes
    were made from."""
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    raw = torch.from_numpy(synth.make_weights(synth.Q4_0, n, k, seed=73)).to(dev)
    vals, scales = ops.separate_blocks(raw, L.Q4_0, n, k)
    plane, scalesT = ops.transpose_q4(vals, n, k), ops.transpose_2d(scales, ldo=(n + 3) // 4 * 4)
    A = torch.from_numpy(synth.make_activations(m, k, 74, np.float16)).to(dev)
    d, C, keep = ops.make_desc(A, plane, L.Q4_0, n, layout=L.LAYOUT_KN_PLANES, scales=scalesT, ldb=plane.stride(0), lds=scalesT.stride(0))
    need = ops.workspace_bytes(d)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    for _ in range(3):
        ops.launch(d)
    torch.cuda.synchronize()
    want = ops.qmatmul(A, raw, L.Q4_0, n)
    rel = float(torch.linalg.norm(C - want) / torch.linalg.norm(want))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(20):
        ops.launch(d)
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) * 1e3 / 20
    return {"us_per_launch": us, "TFLOP/s": 2.0 * m * k * n / us / 1e6, "variant": L.lib().cutb_variant_name(ops.select_variant(d)).decode(),
            "rel_l2_vs_block_gemm": rel}


def projection_shapes_70b():
    """configs[4]: the projections of a 70B-shape decoder layer as (name, N rows, K) of Q4_0 weights."""
    return [("attn_q/o 8192x8192", 8192, 8192), ("ffn_gate/up 28672x8192", 28672, 8192), ("ffn_down 8192x28672", 8192, 28672)]


def secondary_measurements(dev) -> dict:
    """Context numbers for the other benchmark configurations (not the headline value):
    configs[0] Q8_0 4096x4096 fp32 mat-vec (GB/s, weights cycled over 32 copies) and
    configs[2] Q4_K prefill GEMM M=512 K=4096 N=14336 (TFLOP/s = 2 M K N / time), and the
    dequant operator on that weight (GB/s over raw bytes in + fp32 bytes out)."""
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    out = {}

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / iters  # us

    # configs[0]
    n, k, reps = 4096, 4096, 32
    base = torch.from_numpy(synth.make_weights(synth.Q8_0, n, k, seed=31)).to(dev)
    W = torch.stack([torch.roll(base, shifts=34 * 5 * r) for r in range(reps)])
    A = torch.from_numpy(synth.make_activations(1, k, 32, np.float32)).to(dev)
    C = torch.zeros((reps, 1, n), dtype=torch.float32, device=dev)
    descs = [ops.make_desc(A, W[r], L.Q8_0, n, C_out=C[r]) for r in range(reps)]

    def sweep():
        for d, _, _ in descs:
            ops.launch(d)

    sweep()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sweep()
    us = timed(g.replay, 50) / reps
    bytes0 = n * (k // 32) * 34 + k * 4 + n * 4
    out["configs[0]_q8_0_4096x4096_fp32_matvec"] = {"us_per_launch": us, "GB/s": bytes0 / us / 1e3,
                                                      "algorithmic_bytes": bytes0}
    del W, C, descs, g

    # configs[2]
    m, k, n = 512, 4096, 14336
    W = torch.from_numpy(synth.make_weights(synth.Q4_K, n, k, seed=33)).to(dev)
    A = torch.from_numpy(synth.make_activations(m, k, 34, np.float16)).to(dev)
    C = torch.empty((m, n), dtype=torch.float32, device=dev)
    d, _, keep = ops.make_desc(A, W, L.Q4_K, n, C_out=C)
    assert ops.select_variant(d) == L.VARIANT_GEMM_TC
    us = timed(lambda: ops.launch(d), 20)
    flops = 2.0 * m * k * n
    peaks = {}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
    tf = flops / us / 1e6
    out["configs[2]_q4_k_prefill_gemm_512x4096x14336"] = {
        "us_per_launch": us, "TFLOP/s": tf,
        "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"] if "bf16_tflops" in peaks else None,
        "frac_of_measured_bf16_sustained": tf / peaks["bf16_tflops_sustained"] if "bf16_tflops_sustained" in peaks else None,
        "peak_note": "timed alone for 20 launches, so the burst figure is the roofline; the sustained one is for context",
        "kernel": "tcgen05.mma kind::f16, TMEM accumulators"}
    del A, C, d, keep

    # the dequant operator on the same weight (write-bound: 33 MB in, 235 MB out; three output
    # buffers cycled so that L2 cannot absorb the writes)
    outs = [torch.empty((n, k), dtype=torch.float32, device=dev) for _ in range(3)]

    def dq():
        for o in outs:
            ops.dequantize(W, L.Q4_K, n, k, out=o)

    us = timed(dq, 10) / len(outs)
    dq_bytes = W.numel() + n * k * 4
    out["dequant_q4_k_14336x4096"] = {"us_per_launch": us, "GB/s": dq_bytes / us / 1e3, "algorithmic_bytes": dq_bytes,
                                      "frac_of_measured_hbm": (dq_bytes / us / 1e3) / peaks["hbm_gbs"] if "hbm_gbs" in peaks else None}
    del outs, W
    torch.cuda.empty_cache()

    hbm = peaks.get("hbm_gbs")
    # configs[1] at batch 8 (same weight bytes, eight activation rows)
    b8 = chain_us(dev, synth.Q4_0, N_ROWS, K_COLS, 8, np.float16)
    b8["frac_of_measured_hbm"] = b8["GB/s"] / hbm if hbm else None
    out["configs[1]_q4_0_11008x4096_batch8"] = b8
    # the same weight with 16 .. 128 activation rows: what CUTB_VARIANT_AUTO runs there (the mat-vec up to 16 fp16
    # rows, the tensor-core GEMM for up to 128 tokens, the prefill GEMM beyond); bound = the same weight traffic
    for m in (16, 32, 64, 128):
        r = chain_us(dev, synth.Q4_0, N_ROWS, K_COLS, m, np.float16, total_mb=300.0)
        r["frac_of_measured_hbm"] = r["GB/s"] / hbm if hbm else None
        out[f"configs[1]_q4_0_11008x4096_batch{m}"] = r
    # the layout the reference's unchanged loader and runner hand over: [K, N] planes (nibbles [K, N / 2] after its
    # Q4 transpose, fp16 scales [K / 32, N]), batch 1, against the block layout above
    out["configs[1]_q4_0_kn_planes_batch1"] = planes_chain_us(dev, N_ROWS, K_COLS)
    if hbm:
        out["configs[1]_q4_0_kn_planes_batch1"]["frac_of_measured_hbm"] = out["configs[1]_q4_0_kn_planes_batch1"]["GB/s"] / hbm
    out["configs[2]_shape_q4_0_kn_planes_512x4096x14336"] = planes_gemm_us(dev, 512, 4096, 14336)
    # configs[4] on one GPU: the whole 70B-shape projections (the N > 1 runs shard these same tensors)
    proj = {}
    for name, n, k in projection_shapes_70b():
        for m in (1, 8, 32):
            r = chain_us(dev, synth.Q4_0, n, k, m, np.float16, total_mb=400.0)
            r["frac_of_measured_hbm"] = r["GB/s"] / hbm if hbm else None
            proj[f"{name} batch {m}"] = r
    out["configs[4]_70b_q4_0_projections_1gpu"] = proj
    torch.cuda.empty_cache()
    from cut_b200.llama_decode import LlamaConfig, synthetic_weights

    cfg4 = LlamaConfig()
    w4 = synthetic_weights(cfg4, seed=41, distinct_layers=False, scale_shift=7)
    out["configs[3]_llama_q4_k_decode_batch1"] = decode_measurement(dev, weights=w4)
    torch.cuda.empty_cache()
    try:
        out["configs[3]_llama_q4_k_decode_cpp_runner"] = cpp_runner_measurement(dev.index or 0, cfg4, w4)
    except Exception as e:  # noqa: BLE001  (context, never the headline)
        out["configs[3]_llama_q4_k_decode_cpp_runner"] = {"error": f"{type(e).__name__}: {e}"}
    del w4
    return out


def e2e_host_boundary(device: int, base_weights: np.ndarray, a_host_all, steps: int):
    """The same step through the C++ operator API the reference's runner calls (Operations::matmulBlocks recorded
    once into a reusable command buffer; per step ComputeInterface::copyDataToBuffer of every activation from
    pinned host memory, resubmit, wait, copyDataFromBuffer of every result), driven through libcut_host.so's C
    entry.  Returns (seconds, h2d bytes per step, d2h bytes per step, results [REPLICAS, BATCH, N])."""
    import ctypes as C

    import torch

    from cut_b200 import build as B

    lib = C.CDLL(B.build_host())
    f = lib.cut_host_e2e_matvec_blocks
    f.restype = C.c_int
    f.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p,
                  C.c_int, C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                  C.c_char_p, C.c_size_t]
    c_host = torch.empty((REPLICAS, BATCH, N_ROWS), dtype=torch.float32).pin_memory()
    secs, h2d, d2h = C.c_double(0), C.c_uint64(0), C.c_uint64(0)
    err = C.create_string_buffer(512)
    w = np.ascontiguousarray(base_weights)
    rc = f(device, 17, N_ROWS, K_COLS, BATCH, REPLICAS, w.ctypes.data, w.size, 18 * 7, a_host_all.data_ptr(), 1, c_host.data_ptr(), 3,
           steps, C.byref(secs), C.byref(h2d), C.byref(d2h), err, len(err))
    if rc != 0:
        raise SystemExit(f"bench: the C++ operator API failed: {err.value.decode()}")
    return secs.value, h2d.value, d2h.value, c_host


def tp_projection_measurements(dev, rank: int, world: int) -> dict:
    """configs[4] at N > 1: the 70B-shape Q4_0 projections as FIXED tensors row-sharded over the ranks (strong
    scaling: rank r owns rows [r N / g, (r + 1) N / g) of every tensor, activations replicated), with ONE exchange
    per projection, as a decoder needs it (every projection's output feeds the next).  Three ways per shape and batch:
    the local mat-vecs alone, the fused exchange (scatter epilogue + one bounded exchange kernel per projection) and
    an NCCL all-gather per projection.  Batch 32 runs the tensor-core GEMM, which has no scatter epilogue: NCCL only.
    Two output slots alternate: the exchange of projection t + 1 is passed only once every rank has launched it, i.e.
    has consumed projection t's output, so slot t & 1 is free again at t + 2 (a decoder's own data dependence).
    Times are device times of a CUDA-graph chain over distinct weight copies, max over ranks."""
    import torch
    import torch.distributed as dist

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth, tp

    out = {}
    stream_of = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731

    def max_over_ranks(v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, reps: int) -> float:
        """us per projection of `fn` (one pass over `reps` projections), replayed from a CUDA graph."""
        fn()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        iters = max(3, 600 // reps)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        us = max_over_ranks(a.elapsed_time(b) * 1e3 / (iters * reps))
        del g
        return us

    for name, n, k in projection_shapes_70b():
        lo, hi = tp.shard_rows(n, rank, world)
        rows = hi - lo
        rb = synth.row_bytes(synth.Q4_0, k)
        reps = max(2, min(48, int(300e6 // (rows * rb)) + 1))
        base = torch.from_numpy(synth.make_weights(synth.Q4_0, rows, k, seed=400 + rank)).to(dev)
        W = torch.empty((reps, base.numel()), dtype=torch.uint8, device=dev)
        for r in range(reps):
            W[r] = torch.roll(base, shifts=18 * 7 * r)
        for m in (1, 8, 32):
            A = torch.from_numpy(synth.make_activations(m, k, 401, np.float16)).to(dev)
            c_local = torch.zeros((m, rows), dtype=torch.float32, device=dev)
            gathered = torch.zeros((world, m, rows), dtype=torch.float32, device=dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            descs, keep, ws = [], [], None
            for r in range(reps):
                d, _, kp = ops.make_desc(A, W[r], L.Q4_0, rows, C_out=c_local, status=status)
                need = ops.workspace_bytes(d)
                if need:
                    # one scratch block for all copies: the launches are ordered on one stream
                    ws = ws if ws is not None else torch.empty(need, dtype=torch.uint8, device=dev)
                    d.workspace, d.workspace_bytes = ws.data_ptr(), need
                descs.append(d)
                keep.append(kp)
            variant = ops.select_variant(descs[0])
            equal_shards = all(tp.shard_rows(n, q, world)[1] - tp.shard_rows(n, q, world)[0] == rows for q in range(world))

            def local_only():
                for d in descs:
                    ops.launch(d)

            def with_nccl():
                for d in descs:
                    ops.launch(d)
                    dist.all_gather_into_tensor(gathered.view(-1), c_local.view(-1))

            shard_bytes = rows * rb + m * k * 2 + m * rows * 4
            full_bytes = n * rb + m * k * 2 + m * n * 4
            res = {"variant": L.lib().cutb_variant_name(variant).decode(), "rows_per_rank": rows, "weight_copies": reps}
            us = timed(local_only, reps)
            res["no_exchange"] = {"us_per_projection": us, "GB/s_per_gpu": shard_bytes / us / 1e3, "GB/s_aggregate": world * shard_bytes / us / 1e3}
            if equal_shards:
                us = timed(with_nccl, reps)
                res["nccl_all_gather_per_projection"] = {"us_per_projection": us, "GB/s_per_gpu": shard_bytes / us / 1e3,
                                                         "GB/s_aggregate": full_bytes / us / 1e3}
            if variant == L.VARIANT_GEMV_MMA:
                grp = tp.ScatterGroup(m, n, slots=2, device=dev)
                sdescs = []
                for r in range(reps):
                    d, _, kp = ops.make_desc(A, W[r], L.Q4_0, rows, C_out=c_local, status=grp.status, variant=L.VARIANT_GEMV_MMA)
                    if descs[r].workspace:
                        d.workspace, d.workspace_bytes = descs[r].workspace, descs[r].workspace_bytes
                    sdescs.append(d)
                    keep.append(kp)
                peers = [grp.peers(0), grp.peers(1)]

                def with_fused():
                    st = stream_of()
                    for r, d in enumerate(sdescs):
                        grp.launch(d, peers[r & 1], st)
                        grp.exchange(st)

                # parity before timing: the assembled output of the last projection of a pass equals, bit for bit,
                # what mat-vec + all-gather of that projection gives (split-K shapes included)
                with_fused()
                ops.launch(descs[reps - 1])
                dist.all_gather_into_tensor(gathered.view(-1), c_local.view(-1))
                torch.cuda.synchronize()
                ok = True
                if equal_shards:
                    plain = gathered.permute(1, 0, 2).reshape(m, n)
                    ok = bool(torch.equal(plain, grp.out[(reps - 1) & 1])) and int(grp.status.item()) == 0
                flag = torch.tensor([0 if ok else 1], dtype=torch.int32, device=dev)
                dist.all_reduce(flag)
                res["fused_equals_matvec_plus_all_gather_bit_for_bit"] = int(flag.item()) == 0
                if int(flag.item()) == 0:
                    us = timed(with_fused, reps)
                    res["fused_exchange_per_projection"] = {"us_per_projection": us, "GB/s_per_gpu": shard_bytes / us / 1e3,
                                                            "GB/s_aggregate": full_bytes / us / 1e3}
                dist.barrier()
                grp.close()
            out[f"{name} batch {m}"] = res
            del descs, keep, gathered, c_local
        del W, base
        torch.cuda.empty_cache()
    return out


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth, tp

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the quantized-matmul path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L.lib()  # fail loudly if libcutb.so is missing

    # ---- synthetic, device-resident inputs: REPLICAS distinct shards per rank ----
    base = synth.make_weights(synth.Q4_0, N_ROWS, K_COLS, seed=1234 + rank)
    W = torch.empty((REPLICAS, base.size), dtype=torch.uint8, device=dev)
    Wb = torch.from_numpy(base).to(dev)
    for r in range(REPLICAS):
        # distinct bytes per replica without generating 800 MB on the host
        W[r] = torch.roll(Wb, shifts=18 * 7 * r)
    a_host = torch.from_numpy(synth.make_activations(BATCH, K_COLS, 77, np.float16)).pin_memory()
    A = a_host.to(dev)
    C_all = torch.zeros((REPLICAS, BATCH, N_ROWS), dtype=torch.float32, device=dev)
    gathered = torch.zeros((world, REPLICAS, BATCH, N_ROWS), dtype=torch.float32, device=dev) if world > 1 else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    descs, keep = [], []
    for r in range(REPLICAS):
        d, _, k = ops.make_desc(A, W[r], L.Q4_0, N_ROWS, C_out=C_all[r], status=status)
        assert ops.select_variant(d) == L.VARIANT_GEMV_MMA and ops.workspace_bytes(d) == 0
        descs.append(d)
        keep.append(k)

    # N > 1, fused exchange: the epilogue of every mat-vec stores its slice into every rank's full
    # output (peer-mapped), one bounded wait kernel per step orders the stream behind all ranks.
    # Output slots: one per replica, twice (steps that download results alternate between the halves).
    fused = world > 1 and args.exchange == "fused"
    exchange_note = None
    grp = None

    def all_ranks_ok(ok: bool) -> bool:
        t = torch.tensor([0 if ok else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(t)
        return int(t.item()) == 0

    if fused:
        # mapping the peers' buffers can fail on a box without peer access between some pair of
        # GPUs: then every rank takes the NCCL exchange and the line says so
        try:
            grp = tp.ScatterGroup(BATCH, world * N_ROWS, slots=2 * REPLICAS, device=dev)
            ok = True
        except Exception as e:  # noqa: BLE001
            ok, exchange_note = False, f"peer mapping failed on rank {rank}: {e}"
        if not all_ranks_ok(ok):
            fused, grp = False, None
            exchange_note = exchange_note or "peer mapping failed on another rank"
    peer_args = [grp.peers(s) for s in range(2 * REPLICAS)] if fused else None

    def scatter_sweep(ds, half):
        stream = torch.cuda.current_stream().cuda_stream
        for r, d in enumerate(ds):
            grp.launch(d, peer_args[half * REPLICAS + r], stream)
        grp.exchange(stream)

    def sweep():
        if fused:
            scatter_sweep(descs, 0)
            return
        for d in descs:
            ops.launch(d)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), C_all.view(-1))

    # correctness of what is being timed (first rows of replica 0)
    sweep()
    torch.cuda.synchronize()

    # independent of the fused kernel: the (bit-exact, separately tested) dequant operator followed
    # by a float64 dense product on the device, for the first rows of a weight tensor
    rows = 256

    def dense_reference(a_dev, w_bytes_dev):
        wf = ops.dequantize(w_bytes_dev[: rows * (K_COLS // 32) * 18], L.Q4_0, rows, K_COLS).double()
        return (a_dev.double() @ wf.T).cpu().numpy()

    ref = dense_reference(A, W[0])
    if fused:
        got = grp.out[0, :, rank * N_ROWS: rank * N_ROWS + rows].cpu().numpy()
        # and the assembled output equals what the NCCL all-gather of the plain kernel's slices gives
        for d in descs:
            ops.launch(d)
        dist.all_gather_into_tensor(gathered.view(-1), C_all.view(-1))
        torch.cuda.synchronize()
        plain = gathered.permute(1, 2, 0, 3).reshape(REPLICAS, BATCH, world * N_ROWS)
        same = torch.equal(plain, grp.out[:REPLICAS]) and int(grp.status.item()) == 0
        if not all_ranks_ok(same):
            # never time an exchange that does not reproduce mat-vec + all-gather: fall back, and say so
            exchange_note = f"fused exchange failed its check against mat-vec + all-gather (status {int(grp.status.item())})"
            fused = False
            got = C_all[0, :, :rows].cpu().numpy()
    else:
        got = C_all[0, :, :rows].cpu().numpy()
    rel = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
    if not rel <= 1e-3 or int(status.item()) != 0:
        raise SystemExit(f"bench: kernel output disagrees with dense matmul over dequant (rel-L2 {rel}, status {int(status.item())})")

    # ---- device-resident timing: CUDA-graph replay of one sweep per step ----
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        sweep()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            sweep()
        step = graph.replay
    except Exception:
        graph, step = None, sweep

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    bytes_per_launch = algorithmic_bytes(N_ROWS, K_COLS, BATCH)
    launches = REPLICAS * args.steps
    value = world * launches * bytes_per_launch / (ms * 1e-3) / 1e9

    # ---- kernel-only duration for the roofline (no collective), events on the launch stream ----
    def kernels_only():
        for d in descs:
            ops.launch(d)

    g2 = None
    try:
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2):
            kernels_only()
        kstep = g2.replay
    except Exception:
        kstep = kernels_only
    for _ in range(3):
        kstep()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ksteps = max(args.steps, 20)
    k0.record()
    for _ in range(ksteps):
        kstep()
    k1.record()
    torch.cuda.synchronize()
    us_per_launch = k0.elapsed_time(k1) * 1e3 / (ksteps * REPLICAS)
    achieved = bytes_per_launch / (us_per_launch * 1e-6) / 1e9
    peak, peak_kind = measured_peak_gbs()

    # ---- end to end through the host-buffer calls, as the reference's backend is driven: upload
    # the step's inputs (one activation per mat-vec, pinned host memory), the step's dispatches,
    # download the step's results; everything inside the timed region, every step ----
    a_host_all = torch.from_numpy(np.stack([synth.make_activations(BATCH, K_COLS, 77 + r, np.float16)
                                             for r in range(REPLICAS)])).pin_memory()
    A_all = torch.empty_like(a_host_all, device=dev)
    c_host_all = torch.empty((REPLICAS, BATCH, N_ROWS), dtype=torch.float32).pin_memory()
    e2e_descs = []
    for r in range(REPLICAS):
        d, _, k = ops.make_desc(A_all[r], W[r], L.Q4_0, N_ROWS, C_out=C_all[r], status=status)
        e2e_descs.append(d)
        keep.append(k)
    e2e_steps = max(1, min(args.steps, 200))

    def e2e_body(half=0):
        A_all.copy_(a_host_all, non_blocking=True)
        if fused:
            # each rank downloads its own slice of the assembled outputs; consecutive steps use
            # different output halves, so a rank that is one step ahead never writes what another
            # is still downloading
            scatter_sweep(e2e_descs, half)
            c_host_all.copy_(grp.out[half * REPLICAS:(half + 1) * REPLICAS, :, rank * N_ROWS:(rank + 1) * N_ROWS],
                             non_blocking=True)
            return
        for d in e2e_descs:
            ops.launch(d)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), C_all.view(-1))
        c_host_all.copy_(C_all, non_blocking=True)

    e2e_body(0)
    if fused:
        e2e_body(1)
    torch.cuda.synchronize()
    g3 = []
    try:
        for half in ((0, 1) if fused else (0,)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                e2e_body(half)
            g3.append(g)
        e2e_launch = [g.replay for g in g3]
    except Exception:
        g3, e2e_launch = [], [lambda: e2e_body(0), lambda: e2e_body(1)] if fused else [lambda: e2e_body(0)]
    e2e_count = [0]

    def e2e_step():
        e2e_launch[e2e_count[0] % len(e2e_launch)]()
        e2e_count[0] += 1
        torch.cuda.current_stream().synchronize()  # the host reads c_host_all here

    for _ in range(3):
        e2e_step()
    # what came back is what the device-resident path computes for the same inputs
    chk = dense_reference(A_all[REPLICAS - 1], W[REPLICAS - 1])
    rel = float(np.linalg.norm(c_host_all[REPLICAS - 1, :, :rows].numpy() - chk) / np.linalg.norm(chk))
    if not rel <= 1e-3:
        raise SystemExit(f"bench: end-to-end output disagrees with dense matmul over dequant (rel-L2 {rel})")
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * e2e_steps * REPLICAS * bytes_per_launch / e2e_s / 1e9
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": world * a_host_all.numel() * 2,
           "d2h_bytes_per_step": world * c_host_all.numel() * 4, "steps": e2e_steps, "ms_per_step": 1e3 * e2e_s / e2e_steps,
           "graph": bool(g3), "path": "C ABI (cutb_qmatmul) with torch copies: one upload of the step's activations, the step's "
           "mat-vecs, one download of the results, replayed as one CUDA graph"}
    e2e_extra = {}
    if world == 1:
        # N = 1: the headline end-to-end number goes through the boundary the reference's runner calls (the C++ operator
        # API); the C-ABI figure above stays beside it as context
        hs, h2d, d2h, c_hb = e2e_host_boundary(local_rank, base, a_host_all, e2e_steps)
        rel = float(np.linalg.norm(c_hb[REPLICAS - 1, :, :rows].numpy() - chk) / np.linalg.norm(chk))
        if not rel <= 1e-3:
            raise SystemExit(f"bench: the C++ operator API's output disagrees with dense matmul over dequant (rel-L2 {rel})")
        e2e_extra = {"e2e_c_abi_graph": e2e}
        e2e = {"value": e2e_steps * REPLICAS * bytes_per_launch / hs / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": 1e3 * hs / e2e_steps,
               "path": "C++ operator API (Operations::matmulBlocks -> Dispatcher -> B200Compute): per step copyDataToBuffer of "
               "every activation, resubmit of the recorded command buffer, wait, copyDataFromBuffer of every result; inside the "
               "backend the uploads go out as one transfer plus one scatter launch and the results come back as one gather launch "
               "plus one transfer behind the replay"}

    if int(status.item()) != 0:
        raise SystemExit(f"bench: device status word = {int(status.item())}")

    # ---- the other two parts of the metric, as context (rank 0, single GPU only) ----
    extra = {}
    if world == 1:
        extra = secondary_measurements(dev)
    else:
        # decode tok/s at N GPUs: the decoder does not shard (its per-layer exchanges would cost more than the
        # mat-vecs they connect), so every GPU decodes its own batch-1 sequence; time = the slowest rank's
        barrier()
        err = None
        try:
            dm = decode_measurement(dev)
            local = [dm["ms_per_token"] * dm["tokens"], dm["prefill_ms"], -1.0 if dm["logits_finite"] else 0.0, -1.0]
        except Exception as e:  # a rank that fails still joins the reductions below, so nobody waits for it
            err, dm = f"{type(e).__name__}: {e}", None
            local = [float("inf"), float("inf"), 0.0, 0.0]
        t = torch.tensor(local, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # times: slowest rank; flags are stored negated, so MAX is "any rank failed"
        all_ok, all_finite = float(t[3].item()) < 0, float(t[2].item()) < 0
        try:
            extra_tp = {"configs[4]_70b_q4_0_projections_row_sharded": tp_projection_measurements(dev, rank, world)}
        except Exception as e:  # noqa: BLE001  (every rank raises or none: the steps inside are collective)
            extra_tp = {"configs[4]_70b_q4_0_projections_row_sharded": {"error": f"{type(e).__name__}: {e}"}}
        if all_ok and dm is not None:
            extra = {"configs[3]_llama_q4_k_decode_replicas": {
                "mode": "independent replicas: one batch-1 sequence per GPU, no exchange; time = max over ranks",
                "tok/s": world * dm["tokens"] * 1e3 / float(t[0].item()), "tok/s_rank0": dm["tok/s"], "tokens_per_gpu": dm["tokens"],
                "prefill_tok/s": world * 512e3 / float(t[1].item()), "logits_finite": all_finite,
                "kernel_launches_per_token": dm["kernel_launches_per_token"]}}
        else:
            extra = {"configs[3]_llama_q4_k_decode_replicas": {"error": err or "another rank failed"}}
        extra.update(extra_tp)
        barrier()

    cpu = None
    if rank == 0 and world == 1:
        v, cores, sample = cpu_port_throughput(args.cpu_seconds)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "replicas_per_step": REPLICAS,
                "l2": f"{REPLICAS} distinct weight tensors cycled ({REPLICAS * base.size / 1e6:.0f} MB > 126 MB L2)",
                "parallelism": "single GPU" if world == 1 else (
                    f"rows sharded over {world} GPUs, slices exchanged by the mat-vec's peer-store epilogue (NVLink), one bounded exchange kernel per step"
                    if fused else f"rows sharded over {world} GPUs, NCCL all-gather of output slices per step"),
                "graph": graph is not None,
                **({"exchange_note": exchange_note} if exchange_note else {}),
                "pct_of_8TBs": 100.0 * value / world / 8000.0,
                "also_measured": {**extra, **e2e_extra},
            },
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "traffic_source": "ncu capture of this kernel and workload (per launch)",
                         "peak_kind": f"of {peak_kind}",
                         "us_per_launch": us_per_launch, "algorithmic_bytes_per_launch": bytes_per_launch},
            "e2e": e2e,
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the communicator down: with CUDA graphs that captured a collective
        # still alive, destroy_process_group() was seen to block forever on this stack.  Every rank
        # has finished its work and synchronised; the process exit releases the NCCL resources.
        del graph, g2, g3
        torch.cuda.synchronize()
        if grp is not None:
            grp.close()  # unmap the peers' buffers while every rank is still alive
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="budget of the CPU baseline leg")
    ap.add_argument("--decode-only", action="store_true",
                    help="run only the configs[3] decoder measurement on one GPU and print it (not the contract line)")
    ap.add_argument("--decode-layers", type=int, default=32)
    ap.add_argument("--decode-steps", type=int, default=256)
    ap.add_argument("--decode-eager", action="store_true", help="with --decode-only: no CUDA graph (one launch per kernel)")
    ap.add_argument("--decode-synthetic-cache", action="store_true",
                    help="with --decode-only: skip the prompt, fill cache rows 0..511 with synthetic values (profiling aid)")
    ap.add_argument("--exchange", choices=["fused", "nccl"], default="fused",
                    help="N > 1: slices meet through the mat-vec's own peer-store epilogue, or through an NCCL all-gather")
    args = ap.parse_args()
    if args.decode_only:
        import torch

        if not torch.cuda.is_available():
            raise SystemExit("bench: --decode-only needs a CUDA device (there is no CPU path)")
        torch.cuda.set_device(0)
        print(json.dumps({"configs[3]_llama_q4_k_decode_batch1": decode_measurement(
            torch.device("cuda:0"), args.decode_layers, args.decode_steps, graph=not args.decode_eager,
            synthetic_cache=args.decode_synthetic_cache)}), flush=True)
        return
    if args.impl == "reference":
        if args.steps == 2000:
            args.steps, args.warmup = 20, 3
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
