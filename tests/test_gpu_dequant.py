"""GPU parity: cutb_dequant and cutb_transpose_q4 against the golden vectors and
the CPU checker.  Bit-exact (integer / byte work and exact fp32 arithmetic)."""
import numpy as np
import pytest

import refdata as R
from cut_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu

FMTS = [(synth.Q8_0, "q8_0"), (synth.Q4_0, "q4_0"), (synth.Q4_K, "q4_k"), (synth.Q5_K, "q5_k"), (synth.Q6_K, "q6_k"),
        (synth.BF16, "bf16"), (synth.Q4_1, "q4_1"), (synth.Q5_0, "q5_0")]


@pytest.fixture(scope="module")
def gpu():
    import torch

    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from cut_b200 import ops

    return ops


def _dq(gpu, fmt, raw, rows, cols):
    import torch

    from gpu_util import dev

    out = gpu.dequantize(dev(raw), fmt, rows, cols)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("fmt,name", FMTS)
def test_dequant_golden_edge_blocks(gpu, golden, fmt, name):
    raw = golden[f"{name}_edge_raw"]
    want = golden[f"{name}_edge_f32bits"]
    got = _dq(gpu, fmt, raw, 1, want.size)
    assert np.array_equal(got.reshape(-1).view(np.uint32), want)


@pytest.mark.parametrize("fmt,name", FMTS)
def test_dequant_golden_random_blocks(gpu, golden, fmt, name):
    raw = golden[f"{name}_rand_raw"]
    rows, cols = (int(x) for x in golden[f"{name}_rand_shape"])
    got = _dq(gpu, fmt, raw, rows, cols)
    assert np.array_equal(np.ascontiguousarray(got).reshape(-1).view(np.uint32), golden[f"{name}_rand_f32bits"])


@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("rows,cols", [(1, 256), (7, 1280), (4096, 4096), (11008, 4096)])
def test_dequant_matches_checker_bitexact(gpu, fmt, name, rows, cols):
    raw = synth.make_weights(fmt, rows, cols, seed=rows + cols + fmt)
    got = _dq(gpu, fmt, raw, rows, cols)
    want = O.dequant_rows(fmt, raw, rows, cols)
    assert np.array_equal(np.ascontiguousarray(got).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt,cols", [(synth.Q8_0, 32), (synth.Q4_0, 96), (synth.Q8_0, 4064), (synth.BF16, 13), (synth.BF16, 1001)])
def test_dequant_cols_not_multiple_of_eight_octets(gpu, fmt, cols):
    raw = synth.make_weights(fmt, 5, cols, seed=cols)
    got = _dq(gpu, fmt, raw, 5, cols)
    assert np.array_equal(np.ascontiguousarray(got).view(np.uint32), O.dequant_rows(fmt, raw, 5, cols).view(np.uint32))


def test_dequant_q4k_reference_case(gpu):
    # tests/harness/OpRegistry.h:1929-1957
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([R.f16_trunc([1.0])[0]], np.uint16).view(np.uint8)
    blk[4:8] = 1
    blk[12:16] = 1
    i = np.arange(128)
    blk[16:] = ((i % 8) & 0xF) | (((i % 8 + 1) & 0xF) << 4)
    out = _dq(gpu, synth.Q4_K, blk, 1, 256).reshape(-1)
    assert np.all(np.isfinite(out))
    assert np.all(np.abs(out[:32] - (blk[16:48] & 0xF)) <= 0.01)


def test_dequant_rejects_bad_arguments(gpu):
    import torch

    from cut_b200 import _lib as L

    raw = torch.zeros(144, dtype=torch.uint8, device="cuda")
    with pytest.raises(L.CutbError) as e:
        gpu.dequantize(raw, synth.Q4_K, 1, 100)  # cols not a multiple of 256
    assert e.value.status == L.ERR_INVALID
    with pytest.raises(L.CutbError) as e:
        gpu.dequantize(raw, synth.Q4_K, 2, 256)  # raw too small
    assert e.value.status == L.ERR_INVALID
    with pytest.raises(L.CutbError):
        gpu.dequantize(raw, 7, 1, 256)


def test_transpose_q4_reference_case(gpu):
    # tests/runtime/OpCoverageTests.cpp:255-277
    import torch

    from gpu_util import dev

    N = K = 32
    Mv = lambda n, k: (n * K + k) & 0xF
    src = np.zeros((N, K // 2), np.uint8)
    for n in range(N):
        for j in range(K // 2):
            src[n, j] = Mv(n, j) | (Mv(n, j + 16) << 4)
    out = gpu.transpose_q4(dev(src), N, K)
    torch.cuda.synchronize()
    assert tuple(out.shape) == (K, N // 2)
    exp = np.zeros((K, N // 2), np.uint8)
    for k in range(K):
        for n in range(0, N, 2):
            exp[k, n // 2] = Mv(n, k) | (Mv(n + 1, k) << 4)
    assert np.array_equal(out.cpu().numpy(), exp)


@pytest.mark.parametrize("N,K", [(2, 32), (6, 64), (130, 96), (1024, 512), (11008, 4096)])
def test_transpose_q4_matches_checker(gpu, N, K):
    import torch

    from gpu_util import dev

    rng = np.random.default_rng(N * 7 + K)
    stride_in = R.pad4(K // 2)
    src = rng.integers(0, 256, size=(N, stride_in), dtype=np.uint8)
    out = gpu.transpose_q4(dev(src), N, K)
    torch.cuda.synchronize()
    want = O.transpose_q4(src, N, K, stride_in=stride_in, stride_out=R.pad4(N // 2))
    got = out.cpu().numpy()
    assert np.array_equal(got[:, : N // 2], want[:, : N // 2])


def test_transpose_q4_rejects_bad_shapes(gpu):
    import torch

    from cut_b200 import _lib as L

    src = torch.zeros((4, 16), dtype=torch.uint8, device="cuda")
    with pytest.raises(L.CutbError, match="N must be even"):
        gpu.transpose_q4(src, 3, 32)
    with pytest.raises(L.CutbError, match="multiple of 32"):
        gpu.transpose_q4(src, 4, 24)
