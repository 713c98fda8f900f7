"""CPU tests: the checker (oracle/) against the committed golden vectors, the
reference's compiled reader when it is present, and the reference's own
known-answer cases.  No GPU."""
import numpy as np
import pytest

import refdata as R
from cut_b200 import synth
from oracle import oracle as O

FMTS = [(synth.Q8_0, "q8_0"), (synth.Q4_0, "q4_0"), (synth.Q4_K, "q4_k")]
# formats the dequant operator takes: the three above and the rest of the reference's DequantFormat set
DEQ_FMTS = FMTS + [(synth.Q5_K, "q5_k"), (synth.Q6_K, "q6_k"), (synth.BF16, "bf16"), (synth.Q4_1, "q4_1"), (synth.Q5_0, "q5_0")]


@pytest.mark.parametrize("fmt,name", DEQ_FMTS)
def test_dequant_matches_golden_edge_blocks(golden, fmt, name):
    raw = golden[f"{name}_edge_raw"]
    want = golden[f"{name}_edge_f32bits"]
    got = O.dequant(fmt, raw, want.size).view(np.uint32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("fmt,name", DEQ_FMTS)
def test_dequant_matches_golden_random_blocks(golden, fmt, name):
    raw = golden[f"{name}_rand_raw"]
    rows, cols = (int(x) for x in golden[f"{name}_rand_shape"])
    want = golden[f"{name}_rand_f32bits"]
    got = O.dequant_rows(fmt, raw, rows, cols).view(np.uint32).reshape(-1)
    assert np.array_equal(got, want)
    # the generator is deterministic: the fixture's raw bytes are reproducible
    assert np.array_equal(raw, synth.make_weights(fmt, rows, cols, seed=1000 + fmt))


@pytest.mark.parametrize("fmt,name", FMTS[:2])
def test_plane_separation_matches_golden(golden, fmt, name):
    raw = golden[f"{name}_rand_raw"]
    rows, cols = (int(x) for x in golden[f"{name}_rand_shape"])
    vals, scales = (O.q8_separate if fmt == synth.Q8_0 else O.q4_separate)(raw, rows, cols)
    assert np.array_equal(vals.view(np.uint8), golden[f"{name}_rand_sep_values"])
    assert np.array_equal(scales, golden[f"{name}_rand_sep_scales"])


@pytest.mark.skipif(not O.have_ref(), reason="reference reader not built (oracle/_ref)")
@pytest.mark.parametrize("fmt,name", DEQ_FMTS)
@pytest.mark.parametrize("rows,cols", [(1, 256), (3, 512), (16, 4096)])
def test_dequant_matches_compiled_reference(fmt, name, rows, cols):
    raw = synth.make_weights(fmt, rows, cols, seed=rows * 131 + cols + fmt)
    a = O.dequant_rows(fmt, raw, rows, cols)
    b = O.ref_dequant(fmt, raw, rows, cols)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_mt19937_streams_match_golden(golden):
    a = golden["mt19937_42_uniform_0p1_10"]
    assert np.array_equal(R.generate_test_data(a.size), a)
    b = golden["mt19937_42_uniform_m1_1"]
    assert np.array_equal(R.mt19937_uniform(-1.0, 1.0, 42, b.size), b)


def test_f16_helpers():
    # gguf_reader.cpp:515-539 semantics on the interesting bit patterns
    bits = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0xBC00], dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    assert np.array_equal(O.f16_to_f32(bits).view(np.uint32), want.view(np.uint32))
    # the runner's rounding is half-up, the test helper truncates and flushes subnormals
    assert O.f32_to_f16_trunc(1.0) == 0x3C00
    assert O.f32_to_f16_trunc(3e-6) == 0  # subnormal range flushed
    assert O.f32_to_f16_runner(3e-6) == int(np.float32(3e-6).astype(np.float16).view(np.uint16))
    assert O.f32_to_f16_runner(65520.0) == 0x7C00
    x = np.float32(1.0) + np.float32(2.0 ** -11)  # exact tie: half-up rounds away, RNE would keep 0x3C00
    assert O.f32_to_f16_runner(float(x)) == 0x3C01


# ---- the reference's known-answer cases, on the checker's plane-layout matmul ----
def test_q8_simple_and_withscales():
    # OpRegistry.h:1995-2026
    A = np.ones((1, 32), np.float32)
    B = np.tile(np.array([1, 2], np.int8), (32, 1))
    S = R.f16_trunc([1.0, 1.0]).reshape(1, 2)
    c = O.qmatmul_planes(False, False, A, B, S, 1, 32, 2)
    assert abs(c[0, 0] - 32.0) <= 1e-3 and abs(c[0, 1] - 64.0) <= 1e-3
    A = np.ones((1, 64), np.float32)
    B = np.full((64, 2), 4, np.int8)
    S = R.f16_trunc([0.5, 2.0, 1.0, 0.25]).reshape(2, 2)
    c = O.qmatmul_planes(False, False, A, B, S, 1, 64, 2)
    assert abs(c[0, 0] - 192.0) <= 1.0 and abs(c[0, 1] - 288.0) <= 1.0


def test_q4_simple_and_withscales():
    # OpRegistry.h:2054-2086
    A = np.ones((1, 32), np.float32)
    B = np.full((32, 1), R.pack_nibbles(9, 10), np.uint8)
    S = R.f16_trunc([1.0, 1.0]).reshape(1, 2)
    c = O.qmatmul_planes(True, False, A, B, S, 1, 32, 2)
    assert abs(c[0, 0] - 32.0) <= 1e-3 and abs(c[0, 1] - 64.0) <= 1e-3
    A = np.ones((1, 64), np.float32)
    B = np.full((64, 1), R.pack_nibbles(12, 12), np.uint8)
    S = R.f16_trunc([0.5, 2.0, 1.0, 0.25]).reshape(2, 2)
    c = O.qmatmul_planes(True, False, A, B, S, 1, 64, 2)
    assert abs(c[0, 0] - 192.0) <= 1.0 and abs(c[0, 1] - 288.0) <= 1.0


@pytest.mark.parametrize("M,K,N", [(2, 64, 4), (1, 512, 16)])
def test_q8_vsregular(M, K, N):
    # OpRegistry.h:2028-2052, 2118-2152: float triple loop with the un-rounded scales
    A, B, sf, sbits = R.case_q8(M, K, N, "rand")
    got = O.qmatmul_planes(False, False, A, B, sbits, M, K, N)
    ref = np.zeros((M, N), np.float32)
    for m in range(M):
        for n in range(N):
            e = np.float32(0)
            for k in range(K):
                e = np.float32(e + np.float32(np.float32(A[m, k] * np.float32(B[k, n])) * sf[k // 32, n]))
            ref[m, n] = e
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 0.01 + 0.1)


@pytest.mark.parametrize("M,K,N", [(2, 64, 4), (1, 64, 4)])
def test_q4_vsreference(M, K, N):
    # OpRegistry.h:2088-2116, 2154-2192
    A, packed, nib, sf, sbits = R.case_q4(M, K, N, "rand")
    got = O.qmatmul_planes(True, False, A, packed, sbits, M, K, N)
    ref = (A.astype(np.float64) @ ((nib.astype(np.float64) - 8) * np.repeat(sf.astype(np.float64), 32, axis=0)))
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 0.01 + 0.1)


def test_transpose_q4_bitexact_case():
    # tests/runtime/OpCoverageTests.cpp:255-277
    N = K = 32
    Mv = lambda n, k: (n * K + k) & 0xF
    src = np.zeros((N, K // 2), np.uint8)
    for n in range(N):
        for j in range(K // 2):
            src[n, j] = Mv(n, j) | (Mv(n, j + 16) << 4)
    got = O.transpose_q4(src, N, K)
    exp = np.zeros((K, N // 2), np.uint8)
    for k in range(K):
        for n in range(0, N, 2):
            exp[k, n // 2] = Mv(n, k) | (Mv(n + 1, k) << 4)
    assert np.array_equal(got, exp)


def test_dequant_q4k_reference_case():
    # OpRegistry.h:1929-1957: d = 1, dmin = 0, scales 1, first 32 outputs = low nibbles
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([R.f16_trunc([1.0])[0]], np.uint16).view(np.uint8)
    blk[4:8] = 1
    blk[12:16] = 1
    i = np.arange(128)
    blk[16:] = ((i % 8) & 0xF) | (((i % 8 + 1) & 0xF) << 4)
    out = O.dequant(synth.Q4_K, blk, 256)
    assert np.all(np.isfinite(out))
    assert np.all(np.abs(out[:32] - (blk[16:48] & 0xF)) <= 0.01)


def test_block_and_plane_paths_agree():
    """Loader separation + transposes (llama.cpp:942-969, 1000-1021) feed the plane
    kernel the same weights the block path dequantises."""
    N, K = 16, 128
    A = synth.make_activations(3, K, 5)
    w8 = synth.make_weights(synth.Q8_0, N, K, 11)
    vals, sc = O.q8_separate(w8, N, K)
    c_blocks = O.qmatmul_blocks(synth.Q8_0, A, w8, 3, K, N)
    c_planes = O.qmatmul_planes(False, False, A, vals.T.copy(), sc.T.copy(), 3, K, N, acc64=True)
    assert np.array_equal(c_blocks, c_planes)
    w4 = synth.make_weights(synth.Q4_0, N, K, 12)
    packed, sc = O.q4_separate(w4, N, K)
    c_blocks = O.qmatmul_blocks(synth.Q4_0, A, w4, 3, K, N)
    c_planes = O.qmatmul_planes(True, False, A, O.transpose_q4(packed, N, K), sc.T.copy(), 3, K, N, acc64=True)
    assert np.array_equal(c_blocks, c_planes)


def test_q4k_affine_reencode_is_close_not_exact():
    """llama.cpp:573-619: the affine re-encode rounds scale and min to fp16, so the
    reference's own Q4_K matmul differs from the exact dequant by ~1e-4 relative."""
    N, K = 8, 512
    A = synth.make_activations(2, K, 6)
    w = synth.make_weights(synth.Q4_K, N, K, 13)
    packedT, scalesT = O.requant_q4k_affine(w, N, K)
    exact = O.qmatmul_blocks(synth.Q4_K, A, w, 2, K, N)
    affine = O.qmatmul_planes(True, True, A, packedT, scalesT, 2, K, N, acc64=True)
    rel = np.linalg.norm(affine - exact) / np.linalg.norm(exact)
    assert 0 < rel < 1e-3
    with pytest.raises(ValueError):
        O.requant_q4k_affine(w[: 8 * 144], 8, 128 + 64)


def test_epilogue_ops():
    assert O.epilogue(2.0, 1, 133) == pytest.approx(2.0 / (1.0 + np.exp(-2.0)), rel=1e-6)  # SiLU
    assert O.epilogue(-3.0, 1, 130) == 0.0  # ReLU
    assert O.epilogue(2.0, 2, 0, 5.0) == 7.0  # residual add
    assert O.epilogue(2.0, 2, 2, 5.0) == 10.0
    assert O.epilogue(2.0, 0, 0, 5.0) == 2.0


def test_argreduce_replay_equals_the_bit_reversal_rule():
    """The checker replays the reference's 256-thread scan and shared-memory tree literally
    (ReduceArg.cu:27-59); in closed form that prefers, among equal extremes, the smallest
    bit-reversed (i mod 256), then the smallest i."""
    rng = np.random.default_rng(3)
    brev = lambda t: int(f"{t:08b}"[::-1], 2)
    for _ in range(30):
        n = int(rng.integers(1, 3000))
        v = rng.integers(-2, 3, n).astype(np.float32)
        for is_max in (True, False):
            ext = v.max() if is_max else v.min()
            cands = np.flatnonzero(v == ext)
            want = min(cands, key=lambda i: (brev(int(i) % 256), int(i)))
            assert O.argreduce(v, is_max) == float(want)


def test_rmsnorm_and_embedding_checker():
    x = np.arange(1, 9, dtype=np.float32)
    y = O.rmsnorm(x, np.full(8, 2.0, np.float32), 0.0)
    assert np.allclose(y, 2.0 * x / np.sqrt(np.mean(x ** 2)), rtol=1e-6)
    table = np.arange(40, dtype=np.float32).reshape(5, 8)
    assert np.array_equal(O.embedding(np.array([4, 0, 4], np.uint32), table), table[[4, 0, 4]])


# ---- the runner's weight re-encoders (interface/runner/llama/llama.cpp:445-619): the restatements are pinned
# ---- against fixtures that the reference's own functions produced, and against those functions when present
def test_runner_half_conversions_match_golden(golden):
    got = np.array([O.f32_to_f16_runner(float(v)) for v in golden["runner_f32_in"]], dtype=np.uint16)
    assert np.array_equal(got, golden["runner_f32_to_f16"])
    back = O.f16_to_f32(golden["runner_f16_in"]).view(np.uint32)
    want = golden["runner_f16_to_f32_bits"]
    nan = (want & 0x7FFFFFFF) > 0x7F800000  # NaN payloads are not part of the contract
    assert np.array_equal(back[~nan], want[~nan]) and np.all((back[nan] & 0x7FFFFFFF) > 0x7F800000)


def test_runner_q8_0_quantisation_matches_golden(golden):
    vals, scales = O.quantize_rows_q8_0(golden["runner_q8_in"])
    assert np.array_equal(vals.view(np.uint8), golden["runner_q8_values"])
    assert np.array_equal(scales, golden["runner_q8_scales"])


@pytest.mark.parametrize("tag", ["a", "b"])
def test_runner_q4k_affine_reencode_matches_golden(golden, tag):
    n, k = (int(v) for v in golden[f"runner_requant_{tag}_shape"])
    packed, scales = O.requant_q4k_affine(golden[f"runner_requant_{tag}_raw"], n, k)
    assert np.array_equal(packed, golden[f"runner_requant_{tag}_packed"])
    assert np.array_equal(scales, golden[f"runner_requant_{tag}_scales"])


@pytest.mark.skipif(not O.have_ref_runner(), reason="the reference runner helper was not built here")
def test_runner_restatements_match_compiled_reference():
    rr = O.ref_runner()
    rng = np.random.default_rng(99)
    xs = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 12, 20000))).astype(np.float32)
    assert all(O.f32_to_f16_runner(float(v)) == rr.cutref_runner_f32_to_f16(float(v)) for v in xs)
    hs = np.arange(0, 65536, 7, dtype=np.uint16)
    mine = O.f16_to_f32(hs).view(np.uint32)
    ref = np.array([rr.cutref_runner_f16_to_f32(int(h)) for h in hs], dtype=np.float32).view(np.uint32)
    nan = (ref & 0x7FFFFFFF) > 0x7F800000
    assert np.array_equal(mine[~nan], ref[~nan])
    x = (rng.standard_normal(512 * 32) * np.repeat(np.exp(rng.uniform(-14, 8, 512)), 32)).astype(np.float32)
    v0, s0 = O.quantize_rows_q8_0(x)
    v1, s1 = O.ref_runner_quantize_rows_q8_0(x)
    assert np.array_equal(v0, v1) and np.array_equal(s0, s1)
    from cut_b200 import synth

    raw = synth.make_weights(synth.Q4_K, 64, 1024, seed=5)
    p0, q0 = O.requant_q4k_affine(raw, 64, 1024)
    p1, q1 = O.ref_runner_requant_q4k_affine(raw, 64, 1024)
    assert np.array_equal(p0, p1) and np.array_equal(q0, q1)
