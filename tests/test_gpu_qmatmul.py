"""GPU parity: cutb_qmatmul against the CPU checker on the same seeded inputs.

Tolerance: rel-L2 <= 1e-3 against the exact-dequant, double-accumulated
reference (fp32 accumulate on the device); the reference's own per-element
tolerances are used where its tests are replayed."""
import numpy as np
import pytest

import refdata as R
from cut_b200 import _lib as L
from cut_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL = 1e-3
FMTS = [synth.Q8_0, synth.Q4_0, synth.Q4_K]


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    import torch

    assert torch.cuda.is_available(), "these tests need a CUDA device"


def _inputs(fmt, M, K, N, dtype, seed):
    W = synth.make_weights(fmt, N, K, seed)
    A = synth.make_activations(M, K, seed + 1, dtype)
    return A, W


def _ref(fmt, A, W, M, K, N, **kw):
    return O.qmatmul_blocks(fmt, A.astype(np.float32), W, M, K, N, **kw)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("M", [1, 2, 5, 8])
@pytest.mark.parametrize("K,N", [(256, 16), (512, 40), (1024, 1000), (4096, 2368)])
def test_gemv_mma_matches_checker(fmt, dtype, M, K, N):
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(fmt, M, K, N, dtype, seed=M * 1000 + K + N + fmt)
    got, used, st = run_blocks(fmt, A, W, N)
    assert used == L.VARIANT_GEMV_MMA and st == 0
    assert rel_l2(got, _ref(fmt, A, W, M, K, N)) <= TOL


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M,K,N", [(1, 4096, 1024), (1, 14336, 512), (2, 1024, 264), (8, 512, 40), (16, 1024, 264)])
def test_fp32_activations_staged_at_16_bits(fmt, M, K, N):
    """CUTB_FLAG_ACT_16BIT: fp32 activations at one 16-bit level per block (up to 16 rows instead of 8),
    values far outside the fp16 range included: the block scale is fp32."""
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(fmt, M, K, N, np.float32, seed=M + K + fmt)
    A = (A * np.float32(3.0e5)).astype(np.float32)  # > 65504: fp16 activations would overflow
    got, used, st = run_blocks(fmt, A, W, N, flags=L.FLAG_ACT_16BIT)
    assert used == L.VARIANT_GEMV_MMA and st == 0
    ref = _ref(fmt, A, W, M, K, N)
    assert rel_l2(got, ref) <= TOL
    two, _, _ = run_blocks(fmt, A, W, N) if M <= 8 else (None, None, None)
    if two is not None:  # the default two-level staging is the more exact of the two
        assert rel_l2(two, ref) <= rel_l2(got, ref) + 1e-7


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype,flags", [(np.float32, 0), (np.float32, L.FLAG_ACT_16BIT), (np.float16, 0)])
@pytest.mark.parametrize("M,K,N", [(1, 4096, 1024), (3, 1024, 264), (1, 14336, 96), (8, 512, 40)])
def test_fused_rmsnorm_of_the_activations(fmt, dtype, flags, M, K, N):
    """CUTB_FLAG_A_RMSNORM: C = (RMSNorm(A) * weight) . dequant(W)^T in one launch, against the checker's
    RMSNorm followed by its matmul (split-K shapes included: every CTA reduces the whole row)."""
    import torch

    from cut_b200 import ops
    from gpu_util import dev, rel_l2

    A, W = _inputs(fmt, M, K, N, dtype, seed=M * 7 + K + fmt)
    A = (A.astype(np.float32) * 3.0 + 0.5).astype(dtype)
    nw = np.random.default_rng(K).normal(1.0, 0.2, K).astype(np.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    d, C_out, keep = ops.make_desc(dev(A), dev(W), fmt, N, status=status, flags=flags | L.FLAG_A_RMSNORM)
    nwd = dev(nw)
    d.a_norm_weight, d.a_norm_eps = nwd.data_ptr(), 1e-5
    assert ops.select_variant(d) == L.VARIANT_GEMV_MMA
    need = ops.workspace_bytes(d)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    ops.launch(d)
    torch.cuda.synchronize()
    normed = O.rmsnorm(A.astype(np.float32), nw, 1e-5)
    assert int(status.item()) == 0
    assert rel_l2(C_out.cpu().numpy(), _ref(fmt, normed, W, M, K, N)) <= TOL


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M,K,N2", [(1, 4096, 2048), (1, 512, 1200), (3, 1024, 1189), (1, 256, 14336)])
def test_paired_gate_up_rows(fmt, M, K, N2):
    """CUTB_FLAG_GLU_PAIRS: rows (2i, 2i + 1) = (gate_i, up_i), C[m, i] = silu(gate . a) * (up . a), against the
    checker's two matmuls and its SiLU."""
    import torch

    from cut_b200 import ops
    from gpu_util import dev, rel_l2

    A, Wg = _inputs(fmt, M, K, N2, np.float32, seed=K + N2 + fmt)
    Wu = synth.make_weights(fmt, N2, K, seed=K + N2 + fmt + 77)
    rb = synth.row_bytes(fmt, K)
    W = np.stack([Wg.reshape(N2, rb), Wu.reshape(N2, rb)], axis=1).reshape(-1)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    C_out = torch.zeros((M, N2), dtype=torch.float32, device="cuda")
    d, _, keep = ops.make_desc(dev(A), dev(W), fmt, 2 * N2, C_out=C_out, fusion_type=1, fusion_op=133, status=status,
                               flags=L.FLAG_GLU_PAIRS)
    need = ops.workspace_bytes(d)  # no split-K partial sums with paired rows; staged activations from three rows up
    assert (need == 0) == (M < 3)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    ops.launch(d)
    torch.cuda.synchronize()
    g = _ref(fmt, A, Wg, M, K, N2, fusion_type=1, fusion_op=133).astype(np.float64)
    u = _ref(fmt, A, Wu, M, K, N2).astype(np.float64)
    assert int(status.item()) == 0
    assert rel_l2(C_out.cpu().numpy(), (g * u).astype(np.float32)) <= TOL


def test_paired_rows_are_refused_where_no_kernel_has_them():
    from cut_b200 import ops
    from gpu_util import dev

    A, W = _inputs(synth.Q8_0, 64, 512, 128, np.float16, seed=1)  # the any-shape kernel has no paired epilogue
    d, _, keep = ops.make_desc(dev(A), dev(W), synth.Q8_0, 128, fusion_type=1, fusion_op=133, flags=L.FLAG_GLU_PAIRS,
                               variant=L.VARIANT_GENERIC)
    with pytest.raises(L.CutbError) as e:
        ops.launch(d)
    assert e.value.status == 2
    A1, W1 = _inputs(synth.Q8_0, 1, 512, 128, np.float16, seed=1)
    d, _, keep = ops.make_desc(dev(A1), dev(W1), synth.Q8_0, 128, flags=L.FLAG_GLU_PAIRS)  # no unary fusion
    with pytest.raises(L.CutbError) as e:
        ops.launch(d)
    assert e.value.status == 1
    A2, W2 = _inputs(synth.Q8_0, 1, 4096, 128, np.float16, seed=2)  # few rows, long K: the plan splits K
    d, _, keep = ops.make_desc(dev(A2), dev(W2), synth.Q8_0, 128, fusion_type=1, fusion_op=133, flags=L.FLAG_GLU_PAIRS)
    assert ops.workspace_bytes(d) > 0
    with pytest.raises(L.CutbError) as e:
        ops.launch(d)
    assert e.value.status == 2


def test_fused_rmsnorm_needs_the_decode_kernel_and_a_weight():
    import torch

    from cut_b200 import ops
    from gpu_util import dev

    A, W = _inputs(synth.Q8_0, 64, 512, 128, np.float16, seed=1)  # 64 rows: the prefill GEMM would be chosen
    d, _, keep = ops.make_desc(dev(A), dev(W), synth.Q8_0, 128, flags=L.FLAG_A_RMSNORM)
    nw = torch.ones(512, device="cuda")
    d.a_norm_weight, d.a_norm_eps = nw.data_ptr(), 1e-5
    with pytest.raises(L.CutbError) as e:
        ops.launch(d)
    assert e.value.status == 2
    A1, _ = _inputs(synth.Q8_0, 1, 512, 128, np.float16, seed=1)
    d, _, keep = ops.make_desc(dev(A1), dev(W), synth.Q8_0, 128, flags=L.FLAG_A_RMSNORM)
    with pytest.raises(L.CutbError) as e:
        ops.launch(d)
    assert e.value.status == 1


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype,M", [(np.float16, 9), (np.float16, 16), (np.float32, 5), (np.float32, 8)])
def test_gemv_mma_wide_batches(fmt, dtype, M):
    from gpu_util import rel_l2, run_blocks

    K, N = 1024, 264
    A, W = _inputs(fmt, M, K, N, dtype, seed=M + fmt)
    got, used, st = run_blocks(fmt, A, W, N)
    assert used == L.VARIANT_GEMV_MMA and st == 0
    assert rel_l2(got, _ref(fmt, A, W, M, K, N)) <= TOL


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("M,K,N", [(1, 32 * 8, 3), (3, 32 * 24, 37), (33, 512, 64), (2, 4096, 512)])
def test_generic_matches_checker(fmt, dtype, M, K, N):
    from gpu_util import rel_l2, run_blocks

    if fmt == synth.Q4_K and K % 256:
        K = (K // 256 + 1) * 256
    A, W = _inputs(fmt, M, K, N, dtype, seed=M + K + N)
    got, used, st = run_blocks(fmt, A, W, N, variant=L.VARIANT_GENERIC)
    assert used == L.VARIANT_GENERIC
    assert rel_l2(got, _ref(fmt, A, W, M, K, N)) <= TOL


def test_odd_k_routes_to_generic():
    from gpu_util import rel_l2, run_blocks

    M, K, N = 2, 32 * 5, 10  # K not a multiple of 256: no bulk-copy path
    A, W = _inputs(synth.Q4_0, M, K, N, np.float32, seed=3)
    got, used, _ = run_blocks(synth.Q4_0, A, W, N)
    assert used == L.VARIANT_GENERIC
    assert rel_l2(got, _ref(synth.Q4_0, A, W, M, K, N)) <= TOL


# ---- the benchmark configurations at full size ----
def test_config1_q8_0_4096x4096_fp32():
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(synth.Q8_0, 1, 4096, 4096, np.float32, seed=101)
    got, used, st = run_blocks(synth.Q8_0, A, W, 4096)
    assert used == L.VARIANT_GEMV_MMA and st == 0
    assert rel_l2(got, _ref(synth.Q8_0, A, W, 1, 4096, 4096)) <= TOL


@pytest.mark.parametrize("B", [1, 8])
def test_config2_q4_0_11008x4096_fp16(B):
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(synth.Q4_0, B, 4096, 11008, np.float16, seed=202)
    got, used, st = run_blocks(synth.Q4_0, A, W, 11008)
    assert used == L.VARIANT_GEMV_MMA and st == 0
    assert rel_l2(got, _ref(synth.Q4_0, A, W, B, 4096, 11008)) <= TOL


@pytest.mark.parametrize("B", [1, 8])
def test_q4_k_decode_14336x4096_fp16(B):
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(synth.Q4_K, B, 4096, 14336, np.float16, seed=303)
    got, used, st = run_blocks(synth.Q4_K, A, W, 14336)
    assert used == L.VARIANT_GEMV_MMA and st == 0
    assert rel_l2(got, _ref(synth.Q4_K, A, W, B, 4096, 14336)) <= TOL


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype,flags", [(np.float16, 0), (np.float32, 0), (np.float32, L.FLAG_ACT_16BIT), (np.float16, L.FLAG_A_RMSNORM)])
@pytest.mark.parametrize("M,K,N", [(3, 1024, 264), (4, 4096, 2368), (8, 4096, 1000), (16, 2048, 520), (8, 28672, 1024), (5, 8192, 96)])
def test_activations_staged_once_equal_per_block_staging(fmt, dtype, flags, M, K, N):
    """From three activation rows up the decode mat-vec quantises the activations once per call, in a
    launch of its own, into the workspace; with CUTB_FLAG_STAGE_PER_CTA every block does it itself.  The
    two must agree bit for bit (same arithmetic, same layout), on shapes that split K as well, and the
    shared staging must be what cutb_qmatmul_workspace_bytes asks room for."""
    import torch

    from cut_b200 import ops
    from gpu_util import dev, rel_l2

    if dtype == np.float32 and not (flags & L.FLAG_ACT_16BIT) and M > 8:
        pytest.skip("fp32 rows staged at two levels: at most 8 rows in the decode kernel")
    A, W = _inputs(fmt, M, K, N, dtype, seed=900 + M + fmt)
    Ad, Wd = dev(A), dev(W)
    nw = dev(np.random.default_rng(5).uniform(0.5, 1.5, K).astype(np.float32)) if flags & L.FLAG_A_RMSNORM else None
    outs, needs = [], []
    for extra in (0, L.FLAG_STAGE_PER_CTA):
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        d, C_out, keep = ops.make_desc(Ad, Wd, fmt, N, variant=L.VARIANT_GEMV_MMA, status=status, flags=flags | extra)
        if nw is not None:
            d.a_norm_weight, d.a_norm_eps = nw.data_ptr(), 1e-5
        need = ops.workspace_bytes(d)
        needs.append(need)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        d.workspace, d.workspace_bytes = ws.data_ptr(), need
        ops.launch(d)
        ops.launch(d)  # back to back: the second call restages into the same scratch behind the first
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        outs.append(C_out.cpu().numpy())
    assert needs[0] > needs[1]  # the staged activations take workspace
    assert np.array_equal(outs[0], outs[1])
    if not flags & L.FLAG_A_RMSNORM:
        assert rel_l2(outs[0], _ref(fmt, A, W, M, K, N)) <= TOL


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype,M", [(np.float16, 17), (np.float16, 32), (np.float16, 64), (np.float32, 20), (np.float32, 32)])
def test_forced_matvec_runs_row_groups(fmt, dtype, M):
    """CUTB_VARIANT_GEMV_MMA forced beyond one group of activation rows: up to four groups, one after the other, each
    with its own residual rows (binary fusion); refused beyond that.  CUTB_VARIANT_AUTO keeps sending these shapes
    to the GEMM."""
    from gpu_util import rel_l2, run_blocks

    K, N = 1024, 264
    A, W = _inputs(fmt, M, K, N, dtype, seed=M + fmt)
    D = synth.make_activations(M, N, 99)
    got, used, st = run_blocks(fmt, A, W, N, variant=L.VARIANT_GEMV_MMA, D_np=D, fusion_type=2, fusion_op=0)
    assert used == L.VARIANT_GEMV_MMA and st == 0
    assert rel_l2(got, _ref(fmt, A, W, M, K, N, D=D, fusion_type=2, fusion_op=0)) <= TOL
    _, auto, _ = run_blocks(fmt, A, W, N)
    assert auto == L.VARIANT_GEMM_TC
    big = 65 if dtype == np.float16 else 33
    Ab, _ = _inputs(fmt, big, K, N, dtype, seed=1)
    with pytest.raises(L.CutbError) as e:
        run_blocks(fmt, Ab, W, N, variant=L.VARIANT_GEMV_MMA)
    assert e.value.status == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("fmt", FMTS)
def test_long_k_and_few_rows_use_split_k(fmt):
    """70B-shape slices: K = 28672 with N/8 rows per GPU -> K is split across CTAs
    and summed in a fixed order from the workspace."""
    import torch

    from cut_b200 import ops
    from gpu_util import dev, rel_l2, run_blocks

    M, K, N = 8, 28672, 1024
    A, W = _inputs(fmt, M, K, N, np.float16, seed=404 + fmt)
    d, _, keep = ops.make_desc(dev(A), dev(W), fmt, N)
    assert ops.workspace_bytes(d) > 0
    with pytest.raises(L.CutbError) as e:
        ops.launch(d)  # no workspace supplied
    assert e.value.status == L.ERR_WORKSPACE
    got, used, st = run_blocks(fmt, A, W, N)
    assert used == L.VARIANT_GEMV_MMA and st == 0
    assert rel_l2(got, _ref(fmt, A, W, M, K, N)) <= TOL
    got2, _, _ = run_blocks(fmt, A, W, N)
    assert np.array_equal(got, got2)  # deterministic summation order
    torch.cuda.synchronize()


@pytest.mark.parametrize("fmt", FMTS)
def test_gemv_agrees_with_generic_and_is_deterministic(fmt):
    from gpu_util import rel_l2, run_blocks

    M, K, N = 4, 2048, 777
    A, W = _inputs(fmt, M, K, N, np.float16, seed=55)
    a, _, _ = run_blocks(fmt, A, W, N)
    b, _, _ = run_blocks(fmt, A, W, N)
    g, _, _ = run_blocks(fmt, A, W, N, variant=L.VARIANT_GENERIC)
    assert np.array_equal(a, b)
    assert rel_l2(a, g) <= 2e-4  # 16-bit block floating point activations vs exact fp32


@pytest.mark.parametrize("variant", [L.VARIANT_AUTO, L.VARIANT_GENERIC])
@pytest.mark.parametrize("ftype,fop", [(1, 133), (1, 130), (1, 132), (2, 0), (2, 2)])
def test_fused_epilogues(variant, ftype, fop):
    """SiLU / ReLU / GELU and residual add / mul, the epilogues the runner uses
    (interface/runner/llama/llama.cpp:2461; MatMulQ4Common.cuh:63-114)."""
    from gpu_util import run_blocks

    M, K, N = 3, 512, 200
    A, W = _inputs(synth.Q4_0, M, K, N, np.float32, seed=66)
    D = synth.make_activations(M, N, 67) if ftype == 2 else None
    got, _, _ = run_blocks(synth.Q4_0, A, W, N, variant=variant, D_np=D, fusion_type=ftype, fusion_op=fop)
    ref = _ref(synth.Q4_0, A, W, M, K, N, D=D, fusion_type=ftype, fusion_op=fop)
    assert np.allclose(got, ref, rtol=2e-3, atol=2e-4)


UNARY_OPS = [100, 101, 102, 103, 104, 106, 109, 121, 122, 123, 124, 130, 131, 132, 133, 134, 137, 141, 142, 143, 148]
BINARY_OPS = [0, 1, 2, 3, 4, 5, 6, 13, 14]


@pytest.mark.parametrize("variant,M", [(L.VARIANT_GEMV_MMA, 1), (L.VARIANT_GEMV_MMA, 5), (L.VARIANT_GENERIC, 3), (L.VARIANT_GEMM_TC, 40)])
@pytest.mark.parametrize("ftype,fop", [(1, op) for op in UNARY_OPS] + [(2, op) for op in BINARY_OPS])
def test_every_fused_epilogue_op(variant, M, ftype, fop):
    """All 21 unary and 9 binary epilogue operations of the reference (MatMulQ4Common.cuh:63-114) in the decode
    mat-vec (diagonal and shared-k variants), the any-shape kernel and the tensor-core GEMM, against the
    checker's epilogue applied to the checker's matmul.  The kernels' accumulators differ from the checker's in
    the last bits, and several operations are steep or discontinuous (1/x, log, floor, mod, pow), so an output
    passes when it is close to the checker's, or lies within the range the checker's operation takes over
    accumulator +- 2e-3 (relative to max(1, |acc|); 4e-3 for the GEMM, whose weights are rounded to fp16).  NaNs must agree, except within that distance of the edge of an operation's domain
    (sqrt, log, rsqrt of an accumulator next to zero)."""
    from gpu_util import run_blocks

    K, N = 512, 256
    A, W = _inputs(synth.Q8_0, M, K, N, np.float16, seed=300 + fop + 7 * ftype)
    # accumulators of a few units (a power-of-two rescale, exact in fp16): exp and pow stay finite, few sit next to zero
    spread = float(np.std(_ref(synth.Q8_0, A, W, M, K, N)))
    A = (A.astype(np.float32) * np.float32(2.0 ** round(np.log2(1.5 / spread)))).astype(np.float16)
    D = (synth.make_activations(M, N, 301 + fop) * 0.5 + 0.25).astype(np.float32) if ftype == 2 else None
    got, used, st = run_blocks(synth.Q8_0, A, W, N, variant=variant, D_np=D, fusion_type=ftype, fusion_op=fop)
    assert used == variant and st == 0
    acc = _ref(synth.Q8_0, A, W, M, K, N).astype(np.float32)
    # (the tensor-core GEMM rounds its weights to fp16: a wider band)
    delta = (4e-3 if variant == L.VARIANT_GEMM_TC else 2e-3) * np.maximum(1.0, np.abs(acc))

    def apply(x):
        out = np.empty_like(x)
        for i in np.ndindex(x.shape):
            out[i] = O.epilogue(float(x[i]), ftype, fop, float(D[i]) if D is not None else 0.0)
        return out

    with np.errstate(all="ignore"):
        r0 = apply(acc)
        # the operation over the band around the accumulator (kinks and jumps inside it included)
        band = np.stack([apply((acc + t * delta).astype(np.float32)) for t in np.linspace(-1.0, 1.0, 17)])
        lo, hi = np.nanmin(np.where(np.isnan(band), np.inf, band), axis=0), np.nanmax(np.where(np.isnan(band), -np.inf, band), axis=0)
        tol = 1e-4 + 2e-3 * np.abs(r0)
        tol = np.where(np.isfinite(tol), tol, 1e-4)
        near = np.abs(got - r0) <= tol
        step = np.where(np.isfinite(hi - lo), (hi - lo) / 16.0, 0.0)  # what the operation moves between two samples of the band
        between = (got >= lo - tol - step) & (got <= hi + tol + step)
        edge = np.isnan(band).any(axis=0) & ~np.isnan(band).all(axis=0)  # the band crosses the edge of the operation's domain
        both_nan = np.isnan(got) & np.isnan(r0)
        same_inf = np.isinf(got) & (got == r0)
    bad = ~(near | between | both_nan | same_inf | edge)
    assert not bad.any(), (int(bad.sum()), got[bad][:4], r0[bad][:4], acc[bad][:4])
    assert edge.mean() < 0.05


def test_gemm_tc_reports_fp32_activations_beyond_the_fp16_range():
    """The tensor-core GEMM's operand type is fp16: an fp32 activation beyond 65504 would become infinity.  The
    cast kernel reports it through the status word (CUTB_ERR_RANGE) instead of letting it pass silently; the
    same activations are fine for the decode mat-vec (block floating point at fp32 range) and for the any-shape
    kernel."""
    from gpu_util import rel_l2, run_blocks

    M, K, N = 40, 512, 256
    A, W = _inputs(synth.Q8_0, M, K, N, np.float32, seed=808)
    A[7, 100] = 1.0e5
    _, used, st = run_blocks(synth.Q8_0, A, W, N, variant=L.VARIANT_GEMM_TC)
    assert used == L.VARIANT_GEMM_TC and st == L.ERR_RANGE
    got, _, st = run_blocks(synth.Q8_0, A, W, N, variant=L.VARIANT_GENERIC)
    assert st == 0 and rel_l2(got, _ref(synth.Q8_0, A, W, M, K, N)) <= TOL
    got, used, st = run_blocks(synth.Q8_0, A[:8], W, N)
    assert used == L.VARIANT_GEMV_MMA and st == 0 and rel_l2(got, _ref(synth.Q8_0, A[:8], W, 8, K, N)) <= TOL
    A[7, 100] = 6.0e4  # inside the range: no report
    _, _, st = run_blocks(synth.Q8_0, A, W, N, variant=L.VARIANT_GEMM_TC)
    assert st == 0


def test_large_activation_magnitudes_fp32():
    """fp32 activations far outside the fp16 range still contract correctly
    (power-of-two rescale before the hi/lo split)."""
    from gpu_util import rel_l2, run_blocks

    M, K, N = 2, 1024, 64
    A, W = _inputs(synth.Q8_0, M, K, N, np.float32, seed=77)
    A[0] *= 3.0e6
    A[1] *= 2.0e-7
    got, used, _ = run_blocks(synth.Q8_0, A, W, N)
    assert used == L.VARIANT_GEMV_MMA
    ref = _ref(synth.Q8_0, A, W, M, K, N)
    assert rel_l2(got[0], ref[0]) <= TOL and rel_l2(got[1], ref[1]) <= TOL


def test_invalid_descriptors_return_codes():
    import torch

    from cut_b200 import ops
    from gpu_util import dev

    A, W = _inputs(synth.Q4_0, 1, 256, 8, np.float32, seed=1)
    At, Wt = dev(A), dev(W)
    with pytest.raises(L.CutbError) as e:
        ops.qmatmul(At, Wt, synth.Q4_0, 9)  # W too small for N = 9
    assert e.value.status == L.ERR_INVALID
    with pytest.raises(L.CutbError) as e:
        ops.qmatmul(At, Wt, 5, 8)
    assert e.value.status == L.ERR_INVALID
    with pytest.raises(L.CutbError) as e:
        ops.qmatmul(At[:, :100], Wt, synth.Q4_0, 8)  # K not a multiple of 32
    assert e.value.status == L.ERR_INVALID
    with pytest.raises(L.CutbError) as e:
        ops.qmatmul(At, Wt, synth.Q4_0, 8, fusion_type=2)  # binary fusion without D
    assert e.value.status == L.ERR_INVALID
    with pytest.raises(L.CutbError) as e:
        ops.qmatmul(dev(A[:, :32].copy()), Wt, synth.Q4_0, 8, variant=L.VARIANT_GEMV_MMA)  # K = 32: no bulk path
    assert e.value.status == L.ERR_UNSUPPORTED
    with pytest.raises(RuntimeError, match="1D or 2D"):
        ops.qmatmul(torch.zeros((1, 1, 256), device="cuda"), Wt, synth.Q4_0, 8)


# ---- the reference's runtime layout ([K,N] planes) and its known-answer tests ----
def _run_planes(q4, A, B, S, M, K, N, *, affine=False, D=None, ftype=0, fop=0, dtype=np.float32):
    import torch

    from cut_b200 import ops
    from gpu_util import dev

    ldb = R.pad4(N // 2 if q4 else N)
    lds = R.pad4(N)
    Bp = np.zeros((K, ldb), np.uint8)
    Bp[:, : B.shape[1]] = B.view(np.uint8)
    Sp = np.zeros((S.shape[0], lds), np.uint16)
    Sp[:, :N] = S
    out = ops.qmatmul(dev(A.astype(dtype)), dev(Bp), L.Q4_0 if q4 else L.Q8_0, N, layout=L.LAYOUT_KN_PLANES,
                      scales=dev(Sp), affine=affine, ldb=ldb, lds=lds, D=dev(D) if D is not None else None,
                      fusion_type=ftype, fusion_op=fop)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("q4,affine", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (1, 4096, 11008), (2, 2048, 1001), (3, 1024, 264), (4, 512, 38), (1, 96, 8),
                                   (1, 14336, 512)])
def test_plane_layout_matvec_matches_checker_and_anyshape_kernel(q4, affine, dtype, M, K, N):
    """The coalesced mat-vec over the reference's [K, N] planes (one to four rows; K split over warps and,
    for narrow matrices, over blocks with partial sums in the workspace) against the checker's element
    semantics (MatMulQ4Common.cuh:126-153, MatMulQ8Common.cuh:127-200) and against the any-shape kernel on
    the same operands; odd N, strides padded to 4, a K that is not a multiple of 256, the affine mins."""
    import torch

    from cut_b200 import ops
    from gpu_util import dev, rel_l2

    if q4 and N % 2:
        N += 1  # nibble pairs
    rng = np.random.default_rng(K + N + M)
    ldb, lds = R.pad4(N // 2 if q4 else N), R.pad4(N)
    B = rng.integers(0, 256, size=(K, ldb), dtype=np.uint8)
    nsb = K // 32 * (2 if affine else 1)
    S = np.zeros((nsb, lds), np.float16)
    S[: K // 32] = rng.uniform(0.002, 0.02, size=(K // 32, lds)).astype(np.float16)
    if affine:
        S[K // 32:] = rng.uniform(-0.05, 0.05, size=(K // 32, lds)).astype(np.float16)
    A = synth.make_activations(M, K, 5 + M, dtype)
    D = synth.make_activations(M, N, 6 + M)
    want = O.qmatmul_planes(q4, affine, A.astype(np.float32), B, S.view(np.uint16), M, K, N, lda=K, ldb=ldb, lds=lds, acc64=True,
                            D=D, fusion_type=2, fusion_op=0)
    outs = {}
    for variant in (L.VARIANT_GEMV_PLANES, L.VARIANT_GENERIC):
        out = ops.qmatmul(dev(A), dev(B), L.Q4_0 if q4 else L.Q8_0, N, layout=L.LAYOUT_KN_PLANES, scales=dev(S.view(np.uint16)),
                          affine=affine, ldb=ldb, lds=lds, D=dev(D), fusion_type=2, fusion_op=0, variant=variant)
        torch.cuda.synchronize()
        outs[variant] = out.cpu().numpy()
    assert rel_l2(outs[L.VARIANT_GEMV_PLANES], want) <= 1e-5
    assert rel_l2(outs[L.VARIANT_GEMV_PLANES], outs[L.VARIANT_GENERIC]) <= 1e-5
    again = ops.qmatmul(dev(A), dev(B), L.Q4_0 if q4 else L.Q8_0, N, layout=L.LAYOUT_KN_PLANES, scales=dev(S.view(np.uint16)),
                        affine=affine, ldb=ldb, lds=lds, D=dev(D), fusion_type=2, fusion_op=0)
    assert np.array_equal(again.cpu().numpy(), outs[L.VARIANT_GEMV_PLANES])  # the default choice, and deterministic


def test_reference_q8_simple_and_withscales():
    # tests/harness/OpRegistry.h:1995-2026
    c = _run_planes(False, np.ones((1, 32), np.float32), np.tile(np.array([1, 2], np.int8), (32, 1)),
                    R.f16_trunc([1.0, 1.0]).reshape(1, 2), 1, 32, 2)
    assert abs(c[0, 0] - 32.0) <= 1e-3 and abs(c[0, 1] - 64.0) <= 1e-3
    c = _run_planes(False, np.ones((1, 64), np.float32), np.full((64, 2), 4, np.int8),
                    R.f16_trunc([0.5, 2.0, 1.0, 0.25]).reshape(2, 2), 1, 64, 2)
    assert abs(c[0, 0] - 192.0) <= 1.0 and abs(c[0, 1] - 288.0) <= 1.0


def test_reference_q4_simple_and_withscales():
    # tests/harness/OpRegistry.h:2054-2086
    c = _run_planes(True, np.ones((1, 32), np.float32), np.full((32, 1), R.pack_nibbles(9, 10), np.uint8),
                    R.f16_trunc([1.0, 1.0]).reshape(1, 2), 1, 32, 2)
    assert abs(c[0, 0] - 32.0) <= 1e-3 and abs(c[0, 1] - 64.0) <= 1e-3
    c = _run_planes(True, np.ones((1, 64), np.float32), np.full((64, 1), R.pack_nibbles(12, 12), np.uint8),
                    R.f16_trunc([0.5, 2.0, 1.0, 0.25]).reshape(2, 2), 1, 64, 2)
    assert abs(c[0, 0] - 192.0) <= 1.0 and abs(c[0, 1] - 288.0) <= 1.0


@pytest.mark.parametrize("M,K,N", [(2, 64, 4), (1, 512, 16)])
def test_reference_q8_vsregular_and_allvariants(M, K, N):
    # tests/harness/OpRegistry.h:2028-2052, 2118-2152
    A, B, sf, sbits = R.case_q8(M, K, N, "rand")
    got = _run_planes(False, A, B, sbits, M, K, N)
    ref = A.astype(np.float64) @ (B.astype(np.float64) * np.repeat(sf.astype(np.float64), 32, axis=0))
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 0.01 + 0.1)
    assert np.allclose(got, O.qmatmul_planes(False, False, A, B, sbits, M, K, N, acc64=True), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("M,K,N", [(2, 64, 4), (1, 64, 4)])
def test_reference_q4_vsreference_and_allvariants(M, K, N):
    # tests/harness/OpRegistry.h:2088-2116, 2154-2192
    A, packed, nib, sf, sbits = R.case_q4(M, K, N, "rand")
    got = _run_planes(True, A, packed, sbits, M, K, N)
    ref = A.astype(np.float64) @ ((nib.astype(np.float64) - 8) * np.repeat(sf.astype(np.float64), 32, axis=0))
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 0.01 + 0.1)
    assert np.allclose(got, O.qmatmul_planes(True, False, A, packed, sbits, M, K, N, acc64=True), rtol=1e-5, atol=1e-4)


def test_reference_q8_model_geometry_batched_vs_per_row():
    # tests/runtime/RuntimeTests.cpp:2861-2938 (M=4, K=5120, N=4096, fp64 CPU reference)
    M, K, N = 4, 5120, 4096
    A = R.mt19937_uniform(-1.0, 1.0, 42, M * K).reshape(M, K)
    i = np.arange(K * N, dtype=np.int64)
    B = ((i * 7 + 3) % 21 - 10).astype(np.int8).reshape(K, N)
    sf = ((1.0 + (np.arange((K // 32) * N) % 7)) * 0.03125).astype(np.float32).reshape(K // 32, N)
    sbits = sf.astype(np.float16).view(np.uint16)  # exactly representable
    batched = _run_planes(False, A, B, sbits, M, K, N)
    per_row = np.concatenate([_run_planes(False, A[m:m + 1], B, sbits, 1, K, N) for m in range(M)])
    ref = A.astype(np.float64) @ (B.astype(np.float64) * np.repeat(sf.astype(np.float64), 32, axis=0))
    assert np.all(np.abs(batched - ref) <= np.abs(ref) * 2e-3 + 0.05)
    assert np.all(np.abs(batched - per_row) <= np.abs(per_row) * 2e-3 + 0.05)


@pytest.mark.parametrize("M,K,N,silu", [(13, 4096, 5120, False), (13, 5120, 8192, True), (33, 5120, 4096, True)])
def test_reference_q8_ffn_shapes_with_silu(M, K, N, silu):
    # tests/runtime/RuntimeTests.cpp:3054-3118 (N trimmed from 32768 to keep the CPU reference quick)
    A = R.mt19937_uniform(-1.0, 1.0, 42, M * K).reshape(M, K)
    i = np.arange(K * N, dtype=np.int64)
    B = ((i * 7 + 3) % 21 - 10).astype(np.int8).reshape(K, N)
    sf = ((1.0 + (np.arange((K // 32) * N) % 7)) * 0.03125).astype(np.float32).reshape(K // 32, N)
    sbits = sf.astype(np.float16).view(np.uint16)
    got = _run_planes(False, A, B, sbits, M, K, N, ftype=1 if silu else 0, fop=133)
    ref = A.astype(np.float64) @ (B.astype(np.float64) * np.repeat(sf.astype(np.float64), 32, axis=0))
    if silu:
        ref = ref / (1.0 + np.exp(-ref))
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2e-3 + 0.05)


def test_planes_layout_equals_block_layout_through_loader_repack():
    """GGUF blocks -> the loader's plane separation and the load-time repacks
    (gguf_reader.cpp:389-501, TransposeQ4Nibble) -> plane kernel == block kernel."""
    from gpu_util import rel_l2, run_blocks

    N, K, M = 64, 512, 3
    A = synth.make_activations(M, K, 9)
    w8 = synth.make_weights(synth.Q8_0, N, K, 21)
    vals, sc = O.q8_separate(w8, N, K)
    a = _run_planes(False, A, np.ascontiguousarray(vals.T), np.ascontiguousarray(sc.T), M, K, N)
    b, _, _ = run_blocks(synth.Q8_0, A, w8, N)
    assert rel_l2(a, b) <= 1e-5
    w4 = synth.make_weights(synth.Q4_0, N, K, 22)
    packed, sc = O.q4_separate(w4, N, K)
    a = _run_planes(True, A, O.transpose_q4(packed, N, K), np.ascontiguousarray(sc.T), M, K, N)
    b, _, _ = run_blocks(synth.Q4_0, A, w4, N)
    assert rel_l2(a, b) <= 1e-5


def test_affine_q4_planes_from_q4k():
    """The runner's Q4_K -> affine re-encode (llama.cpp:573-619) through the plane kernel."""
    from gpu_util import rel_l2

    N, K, M = 32, 512, 2
    A = synth.make_activations(M, K, 10)
    w = synth.make_weights(synth.Q4_K, N, K, 23)
    packedT, scalesT = O.requant_q4k_affine(w, N, K)
    got = _run_planes(True, A, packedT, scalesT, M, K, N, affine=True)
    assert rel_l2(got, O.qmatmul_planes(True, True, A, packedT, scalesT, M, K, N, acc64=True)) <= 1e-5
    assert rel_l2(got, _ref(synth.Q4_K, A, w, M, K, N)) <= TOL


# ---- prefill GEMM on the tcgen05 tensor cores ----
@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("M,K,N", [(17, 256, 128), (64, 1024, 136), (128, 512, 1000), (200, 768, 264), (512, 1024, 384),
                                   (300, 512, 256),   # three token blocks: one 256-token pair and one 128-token MMA
                                   (600, 512, 130),   # two CTAs along the tokens, the second mostly zero-filled
                                   (1100, 256, 72)])  # three CTAs along the tokens, one partial weight tile
def test_gemm_tc_matches_checker(fmt, dtype, M, K, N):
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(fmt, M, K, N, dtype, seed=M + K + N + fmt)
    got, used, st = run_blocks(fmt, A, W, N)
    assert used == L.VARIANT_GEMM_TC and st == 0
    # fp16 operands (activations and dequantised weights), fp32 accumulate in tensor memory
    assert rel_l2(got, _ref(fmt, A, W, M, K, N)) <= TOL


@pytest.mark.parametrize("fmt,dtype,M,K,N", [
    (synth.Q4_0, np.float16, 32, 4096, 11008),   # 43 tiles of 256 rows over the SMs: most CTAs end one tile and begin the next
    (synth.Q8_0, np.float32, 33, 1024, 25600),   # 100 tiles, runs of 3 units of a tile's 4
    (synth.Q4_K, np.float16, 128, 2048, 1024),   # few tiles, many CTAs per tile; all 128 tokens
    (synth.Q4_0, np.float16, 24, 256, 38400),    # more tiles than SMs: no split, one unit per tile
    (synth.Q4_K, np.float32, 5, 512, 700),       # a last tile that ends inside its third granule
    (synth.Q4_0, np.float16, 96, 1024, 18944)])  # 65..128 tokens with enough 128-row tiles: the prefill kernel
def test_gemm_tc_splits_k_stages_over_the_sms(fmt, dtype, M, K, N):
    """Up to 128 tokens (tokens = MMA M operand, 256 weight rows = N operand) the 256-k units of all weight tiles
    are dealt evenly to the SMs; a tile shared by several CTAs is summed from their workspace slots in a fixed
    order, with the fused op applied after the sum."""
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(fmt, M, K, N, dtype, seed=M + N)
    D = synth.make_activations(M, N, 5)
    got, used, st = run_blocks(fmt, A, W, N, D_np=D, fusion_type=2, fusion_op=0, variant=L.VARIANT_GEMM_TC)
    assert used == L.VARIANT_GEMM_TC and st == 0
    rb = synth.row_bytes(fmt, K)
    for lo, hi in ((0, 300), (N // 2 - 150, N // 2 + 150), (N - 300, N)):
        ref = _ref(fmt, A, W[lo * rb:hi * rb], M, K, hi - lo, D=np.ascontiguousarray(D[:, lo:hi]), fusion_type=2, fusion_op=0)
        assert rel_l2(got[:, lo:hi], ref) <= TOL
    again, _, _ = run_blocks(fmt, A, W, N, D_np=D, fusion_type=2, fusion_op=0, variant=L.VARIANT_GEMM_TC)
    assert np.array_equal(got, again)  # fixed summation order


@pytest.mark.parametrize("fmt,dtype,M,K,N", [
    (synth.Q4_K, np.float16, 40, 1024, 1000),    # the GEMM for few tokens, K split over the SMs (fix-up pairs the columns)
    (synth.Q4_0, np.float32, 24, 256, 38400),    # the same with whole tiles (the kernel's own epilogue pairs them)
    (synth.Q8_0, np.float16, 100, 512, 33000),   # 65..128 tokens on enough tiles: the prefill kernel
    (synth.Q4_K, np.float16, 300, 512, 264)])    # the prefill kernel, three token blocks
def test_paired_gate_up_rows_in_the_gemm_epilogues(fmt, dtype, M, K, N):
    """CUTB_FLAG_GLU_PAIRS on the tensor-core GEMMs: C[m, i] = SiLU(acc[m, 2i]) * acc[m, 2i + 1], N / 2 output columns."""
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(fmt, M, K, N, dtype, seed=M + N)
    got, used, st = run_blocks(fmt, A, W, N, fusion_type=1, fusion_op=133, flags=L.FLAG_GLU_PAIRS)
    assert used == L.VARIANT_GEMM_TC and st == 0
    assert got.shape == (M, N // 2)
    rb = synth.row_bytes(fmt, K)
    for lo, hi in ((0, 256), (N - 256, N)):
        acc = _ref(fmt, A, W[lo * rb:hi * rb], M, K, hi - lo).astype(np.float64)
        want = acc[:, 0::2] / (1.0 + np.exp(-acc[:, 0::2])) * acc[:, 1::2]
        assert rel_l2(got[:, lo // 2:hi // 2], want) <= 2 * TOL


@pytest.mark.parametrize("fmt,dtype,M,K,N,glu", [
    (synth.Q4_K, np.float16, 512, 8192, 1024, False),   # 8 weight tiles, K shared out eight ways
    (synth.Q4_0, np.float32, 600, 8192, 520, False),    # two token groups, a ragged last tile, the fp16 copy in front
    (synth.Q8_0, np.float16, 512, 14336, 512, True)])   # paired rows finished by the reduction
def test_gemm_tc_splits_a_long_k_over_ctas(fmt, dtype, M, K, N, glu):
    """512 tokens and more on few weight rows with K >= 8192: the K stages are shared out over blockIdx.z, the planes of
    partial sums are added in a fixed order and the fused op follows the sum."""
    from gpu_util import rel_l2, run_blocks

    A, W = _inputs(fmt, M, K, N, dtype, seed=M + K)
    if glu:
        got, used, st = run_blocks(fmt, A, W, N, fusion_type=1, fusion_op=133, flags=L.FLAG_GLU_PAIRS)
        acc = _ref(fmt, A, W, M, K, N).astype(np.float64)
        want = acc[:, 0::2] / (1.0 + np.exp(-acc[:, 0::2])) * acc[:, 1::2]
        tol = 2 * TOL
    else:
        D = synth.make_activations(M, N, 7)
        got, used, st = run_blocks(fmt, A, W, N, D_np=D, fusion_type=2, fusion_op=0)
        want = _ref(fmt, A, W, M, K, N, D=D, fusion_type=2, fusion_op=0)
        tol = TOL
    assert used == L.VARIANT_GEMM_TC and st == 0
    assert rel_l2(got, want) <= tol


def test_thirteen_to_sixteen_rows_on_a_large_weight_take_the_gemm():
    """The automatic choice: up to 12 fp16 rows, small weights and fp32 rows stay on the mat-vec; 13 to 16 fp16 rows on
    16 M weights and more go to the tensor-core GEMM for few tokens."""
    from gpu_util import rel_l2, run_blocks

    K, N = 4096, 4096
    for M, want in ((12, L.VARIANT_GEMV_MMA), (13, L.VARIANT_GEMM_TC), (16, L.VARIANT_GEMM_TC)):
        A, W = _inputs(synth.Q4_K, M, K, N, np.float16, seed=M)
        got, used, st = run_blocks(synth.Q4_K, A, W, N)
        assert used == want and st == 0
        ref = _ref(synth.Q4_K, A, W[:256 * synth.row_bytes(synth.Q4_K, K)], M, K, 256)
        assert rel_l2(got[:, :256], ref) <= TOL
    A, W = _inputs(synth.Q4_K, 8, K, N, np.float32, seed=3)
    _, used, _ = run_blocks(synth.Q4_K, A, W, N)
    assert used == L.VARIANT_GEMV_MMA


def test_gemm_tc_without_room_for_the_split_runs_one_tile_per_cta():
    import torch
    from cut_b200 import ops
    from gpu_util import dev, rel_l2

    M, K, N = 48, 1024, 1280
    A_np, W_np = _inputs(synth.Q4_0, M, K, N, np.float16, seed=12)
    d, C_out, keep = ops.make_desc(dev(A_np), dev(W_np), synth.Q4_0, N, variant=L.VARIANT_GEMM_TC)
    assert ops.workspace_bytes(d) > 0  # the split's slots
    ops.launch(d)  # no workspace given
    torch.cuda.synchronize()
    assert rel_l2(C_out.cpu().numpy(), _ref(synth.Q4_0, A_np, W_np, M, K, N)) <= TOL


@pytest.mark.parametrize("ftype,fop", [(1, 133), (2, 0)])
def test_gemm_tc_fused_epilogues(ftype, fop):
    from gpu_util import run_blocks

    M, K, N = 96, 512, 200
    A, W = _inputs(synth.Q4_K, M, K, N, np.float16, seed=88)
    D = synth.make_activations(M, N, 89) if ftype == 2 else None
    got, used, _ = run_blocks(synth.Q4_K, A, W, N, D_np=D, fusion_type=ftype, fusion_op=fop)
    assert used == L.VARIANT_GEMM_TC
    ref = _ref(synth.Q4_K, A, W, M, K, N, D=D, fusion_type=ftype, fusion_op=fop)
    from gpu_util import rel_l2

    assert rel_l2(got, ref) <= 2e-3  # fp16 operands feed the epilogue: same tolerance class as the unfused GEMM


def test_gemm_tc_agrees_with_generic_on_fp16_rounded_weights():
    """Q8_0 / Q4_0 weights times fp16 scales are formed in fp16 as the reference's tensor-core
    variants do; against the exact-fp32 SIMT variant the difference stays at fp16 rounding level."""
    from gpu_util import rel_l2, run_blocks

    M, K, N = 48, 1024, 256
    for fmt in FMTS:
        A, W = _inputs(fmt, M, K, N, np.float16, seed=5 + fmt)
        a, used, _ = run_blocks(fmt, A, W, N)
        g, _, _ = run_blocks(fmt, A, W, N, variant=L.VARIANT_GENERIC)
        assert used == L.VARIANT_GEMM_TC
        assert rel_l2(a, g) <= 6e-4


def test_config3_q4_k_prefill_512x4096x14336():
    """Benchmark configuration 3 at full size; the CPU checker covers the first and last 192 weight rows."""
    from gpu_util import rel_l2, run_blocks

    M, K, N = 512, 4096, 14336
    A, W = _inputs(synth.Q4_K, M, K, N, np.float16, seed=303)
    got, used, st = run_blocks(synth.Q4_K, A, W, N)
    assert used == L.VARIANT_GEMM_TC and st == 0
    rb = synth.row_bytes(synth.Q4_K, K)
    for lo, hi in ((0, 192), (N - 192, N)):
        ref = _ref(synth.Q4_K, A, W[lo * rb:hi * rb], M, K, hi - lo)
        assert rel_l2(got[:, lo:hi], ref) <= TOL
    assert np.all(np.isfinite(got))


# ---- size-independent properties at the benchmark configurations' full sizes ----
@pytest.mark.parametrize("fmt,M,K,N", [(synth.Q8_0, 1, 4096, 4096), (synth.Q4_0, 1, 4096, 11008), (synth.Q4_0, 8, 4096, 11008),
                                       (synth.Q4_K, 512, 4096, 14336)])
def test_full_size_matmul_equals_dense_matmul_over_dequant(fmt, M, K, N):
    """Every output of the fused kernels against an independent composition on the device: the
    (bit-exact, separately tested) dequant operator followed by a float64 dense matmul."""
    import torch

    from cut_b200 import ops
    from gpu_util import dev

    A, W = _inputs(fmt, M, K, N, np.float16, seed=7 * M + fmt)
    a_d, w_d = dev(A), dev(W)
    got = ops.qmatmul(a_d, w_d, fmt, N)
    dense = ops.dequantize(w_d, fmt, N, K).double()
    ref = a_d.double() @ dense.T
    torch.cuda.synchronize()
    rel = float(torch.linalg.norm(got.double() - ref) / torch.linalg.norm(ref))
    assert rel <= TOL
    assert bool(torch.isfinite(got).all())


@pytest.mark.parametrize("fmt,M,K,N", [(synth.Q4_0, 1, 4096, 11008), (synth.Q4_K, 512, 4096, 14336)])
def test_full_size_linearity_in_the_activations(fmt, M, K, N):
    import torch

    from cut_b200 import ops
    from gpu_util import dev

    x, W = _inputs(fmt, M, K, N, np.float16, seed=11 + fmt)
    y = synth.make_activations(M, K, 99, np.float16)
    w_d = dev(W)
    xd, yd = dev(x), dev(y)
    comb = (2.0 * xd.float() - 3.0 * yd.float()).half()
    lhs = ops.qmatmul(comb, w_d, fmt, N).double()
    # the combination was rounded to fp16: compare against the same rounded vector's decomposition
    rhs = 2.0 * ops.qmatmul(xd, w_d, fmt, N).double() - 3.0 * ops.qmatmul(yd, w_d, fmt, N).double()
    torch.cuda.synchronize()
    rel = float(torch.linalg.norm(lhs - rhs) / torch.linalg.norm(rhs))
    assert rel <= 2e-3  # two extra fp16 roundings of the combined activations on top of the kernel's own tolerance
