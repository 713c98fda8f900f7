"""GPU parity of the load-time repacks: block separation, plane transposes, the Q4_K -> affine
re-encode and the Q8_0 requantiser, each bit for bit against the CPU checker (which is pinned
against the reference's compiled reader where the reference has that code on the CPU side)."""
import numpy as np
import pytest

from cut_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import torch

    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from cut_b200 import ops

    return ops


def _dev(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("fmt,name", [(synth.Q8_0, "q8_0"), (synth.Q4_0, "q4_0")])
def test_separate_matches_golden_planes(gpu, golden, fmt, name):
    raw = golden[f"{name}_rand_raw"]
    rows, cols = (int(x) for x in golden[f"{name}_rand_shape"])
    vals, scales = gpu.separate_blocks(_dev(raw), fmt, rows, cols)
    assert np.array_equal(vals.cpu().numpy().view(np.uint8).reshape(-1), golden[f"{name}_rand_sep_values"].reshape(-1))
    assert np.array_equal(scales.cpu().numpy().view(np.uint16), golden[f"{name}_rand_sep_scales"])


@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_0])
@pytest.mark.parametrize("rows,cols", [(1, 32), (5, 96), (64, 4096), (11008, 4096)])
def test_separate_matches_checker(gpu, fmt, rows, cols):
    raw = synth.make_weights(fmt, rows, cols, seed=rows + cols)
    vals, scales = gpu.separate_blocks(_dev(raw), fmt, rows, cols)
    wv, ws = (O.q8_separate if fmt == synth.Q8_0 else O.q4_separate)(raw, rows, cols)
    assert np.array_equal(vals.cpu().numpy().view(np.uint8), wv.view(np.uint8))
    assert np.array_equal(scales.cpu().numpy().view(np.uint16), ws)


@pytest.mark.parametrize("dtype", [np.int8, np.uint16])
@pytest.mark.parametrize("R,C,pad", [(1, 1, 0), (33, 65, 3), (4096, 128, 0), (300, 11008, 4)])
def test_transpose_2d(gpu, dtype, R, C, pad):
    rng = np.random.default_rng(R * 7 + C)
    x = rng.integers(0, 127, size=(R, C)).astype(dtype)
    out = gpu.transpose_2d(_dev(x.view(np.int8) if dtype == np.int8 else x.view(np.int16)), ldo=R + pad).cpu().numpy()
    out = out.view(dtype)
    assert np.array_equal(out[:, :R], x.T)
    assert not out[:, R:].any()


@pytest.mark.parametrize("N,K", [(2, 256), (6, 512), (64, 4096), (1000, 1024)])
def test_requant_q4k_affine_bitexact(gpu, N, K):
    raw = synth.make_weights(synth.Q4_K, N, K, seed=N + K)
    packedT, scalesT = gpu.requant_q4k_affine(_dev(raw), N, K)
    wp, ws = O.requant_q4k_affine(raw, N, K)
    assert np.array_equal(packedT.cpu().numpy(), wp)
    assert np.array_equal(scalesT.cpu().numpy().view(np.uint16), ws)


def test_requant_q4k_affine_feeds_the_plane_matmul(gpu):
    """The device-side re-encode produces operands the affine plane kernel accepts: same result as
    with the CPU-side re-encode."""
    import torch

    from cut_b200 import _lib as L

    M, K, N = 3, 512, 64
    raw = synth.make_weights(synth.Q4_K, N, K, seed=5)
    A = synth.make_activations(M, K, 6)
    packedT, scalesT = gpu.requant_q4k_affine(_dev(raw), N, K)
    wp, ws = O.requant_q4k_affine(raw, N, K)
    ref = O.qmatmul_planes(True, True, A, wp, ws, M, K, N)
    ref_dev = O.qmatmul_planes(True, True, A, packedT.cpu().numpy(), scalesT.cpu().numpy().view(np.uint16), M, K, N)
    assert np.array_equal(ref, ref_dev)
    torch.cuda.synchronize()
    assert L.OK == 0


def test_requant_rejects_what_the_reference_declines(gpu):
    from cut_b200 import _lib as L

    raw = _dev(synth.make_weights(synth.Q4_K, 3, 256, seed=1))
    with pytest.raises(L.CutbError) as e:
        gpu.requant_q4k_affine(raw, 3, 256)  # odd N
    assert e.value.status == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("n", [96, 4096, 32 * 1000 + 32])
def test_quantize_rows_q8_0_bitexact(gpu, n):
    rng = np.random.default_rng(n)
    x = rng.normal(0, 1, n).astype(np.float32)
    x[:32] = 0.0                      # an all-zero block: d = 0, q = 0
    x[40] = 127.0                     # a block whose maximum is exactly representable
    x[70:74] = [0.5, -0.5, 1.5, -1.5]  # ties of lround
    vals, scales = gpu.quantize_rows_q8_0(_dev(x))
    wv, ws = O.quantize_rows_q8_0(x)
    assert np.array_equal(vals.cpu().numpy(), wv)
    assert np.array_equal(scales.cpu().numpy().view(np.uint16), ws)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [synth.Q6_K, synth.Q5_K, synth.Q4_1, synth.Q5_0, synth.Q4_K])
def test_requant_to_q8_0_blocks_is_the_runners_requantisation(fmt):
    """The runner turns the formats its matmul does not take into Q8_0 at load time: dequantise (exact), then
    quantizeRowsQ8_0 (interface/runner/llama/llama.cpp:488-505, 750-767).  The device does both in one kernel and
    writes GGUF Q8_0 blocks: byte-exact against the checker's composition, and the mat-vec over those blocks
    agrees with the dense product over the original weights to the accuracy of an 8-bit re-encode."""
    import torch

    from cut_b200 import ops
    from oracle import oracle as O

    rows, cols = 24, 1024
    raw = synth.make_weights(fmt, rows, cols, seed=70 + fmt)
    w = O.dequant_rows(fmt, raw, rows, cols)
    vals, scales = O.quantize_rows_q8_0(w.reshape(-1))
    want = np.zeros((rows * cols // 32, 34), dtype=np.uint8)
    want[:, 0:2] = scales.view(np.uint8).reshape(-1, 2)
    want[:, 2:] = vals.view(np.uint8).reshape(-1, 32)
    got = ops.requant_q8_0_blocks(torch.from_numpy(raw).cuda(), fmt, rows, cols)
    assert np.array_equal(got.cpu().numpy(), want.reshape(-1))
    a = synth.make_activations(1, cols, 3, np.float32)
    out = ops.qmatmul(torch.from_numpy(a).cuda(), got, synth.Q8_0, rows).cpu().numpy()
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    assert np.linalg.norm(out - ref) / np.linalg.norm(ref) < 1e-2
