"""GPU parity of the layer operators next to the matmul: RMSNorm within 1e-5 (fp32) / fp16
rounding of the CPU checker, embedding gather and arg-reduce exact, ties included."""
import numpy as np
import pytest

from cut_b200 import _lib as L
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


@pytest.mark.parametrize("rows,dim", [(1, 4), (1, 4096), (7, 100), (512, 4096), (3, 8192 + 12)])
def test_rmsnorm_fp32(gpu, rows, dim):
    rng = np.random.default_rng(rows * 31 + dim)
    x = rng.normal(0, 2.0, (rows, dim)).astype(np.float32)
    w = rng.normal(1.0, 0.1, dim).astype(np.float32)
    y = gpu.rmsnorm(_dev(x), _dev(w), 1e-5).cpu().numpy()
    ref = O.rmsnorm(x, w, 1e-5)
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) <= 1e-6  # fp32 sum of squares against a float64 one
    assert np.max(np.abs(y - ref)) <= 1e-5 * max(1.0, float(np.max(np.abs(ref))))


def test_rmsnorm_reference_case(gpu):
    # tests/harness/OpRegistry.h: x = 1..dim, weight = 1: y = x / sqrt(mean(x^2) + eps)
    dim = 64
    x = np.arange(1, dim + 1, dtype=np.float32)
    y = gpu.rmsnorm(_dev(x), _dev(np.ones(dim, np.float32)), 1e-5).cpu().numpy()
    want = x / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5)
    assert np.allclose(y, want, rtol=1e-5, atol=1e-6)


def test_rmsnorm_fp16(gpu):
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1.0, (9, 4096)).astype(np.float16)
    w = rng.normal(1.0, 0.1, 4096).astype(np.float16)
    y = gpu.rmsnorm(_dev(x), _dev(w), 1e-5).cpu().numpy().astype(np.float32)
    ref = O.rmsnorm(x.astype(np.float32), w.astype(np.float32), 1e-5)
    assert np.max(np.abs(y - ref)) <= 2e-3 * max(1.0, float(np.max(np.abs(ref))))  # one fp16 rounding of the result


@pytest.mark.parametrize("vocab,dim,n", [(10, 4, 3), (32000, 4096, 512), (100, 5, 17)])
def test_embedding_gather_exact(gpu, vocab, dim, n):
    rng = np.random.default_rng(vocab + dim)
    ld = (dim + 3) // 4 * 4
    table = rng.normal(0, 0.02, (vocab, ld)).astype(np.float32)
    idx = rng.integers(0, vocab, n).astype(np.int32)
    out = gpu.embedding(_dev(idx), _dev(table), dim).cpu().numpy()
    assert np.array_equal(out, O.embedding(idx.astype(np.uint32), table))


def test_embedding_index_past_the_table_is_reported_not_read(gpu):
    import torch

    from cut_b200 import _lib as L

    table = _dev(np.ones((4, 8), np.float32))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = gpu.embedding(_dev(np.array([1, 9, 2], np.int32)), table, 8, status=status).cpu().numpy()
    assert int(status.item()) == L.ERR_INVALID
    assert np.array_equal(out[0], np.ones(8)) and not out[1].any() and np.array_equal(out[2], np.ones(8))


@pytest.mark.parametrize("is_max", [True, False])
@pytest.mark.parametrize("n", [1, 255, 256, 1000, 32000, 128256])
def test_argreduce_random(gpu, is_max, n):
    rng = np.random.default_rng(n + int(is_max))
    v = rng.normal(0, 1, n).astype(np.float32)
    got = float(gpu.argreduce(_dev(v), is_max).cpu().numpy()[0])
    assert got == O.argreduce(v, is_max)
    assert got == float(np.argmax(v) if is_max else np.argmin(v))


@pytest.mark.parametrize("is_max", [True, False])
def test_argreduce_ties_follow_the_reference_tree(gpu, is_max):
    rng = np.random.default_rng(77)
    for trial in range(20):
        n = int(rng.integers(300, 5000))
        v = rng.integers(-3, 4, n).astype(np.float32)  # many ties
        got = float(gpu.argreduce(_dev(v), is_max).cpu().numpy()[0])
        assert got == O.argreduce(v, is_max), (trial, n)
    for n in (8192, 32000, 40001):  # long inputs: eight blocks as one cluster
        v = rng.integers(-3, 4, n).astype(np.float32)
        got = float(gpu.argreduce(_dev(v), is_max).cpu().numpy()[0])
        assert got == O.argreduce(v, is_max), n
    # the classic trap: the lowest index does not win
    v = np.zeros(1000, np.float32)
    v[1] = v[128] = 5.0 if is_max else -5.0
    assert float(gpu.argreduce(_dev(v), is_max).cpu().numpy()[0]) == O.argreduce(v, is_max) == 128.0


def test_argreduce_of_nothing_better_than_the_start_value(gpu):
    v = np.full(100, -3.402823466e+38, np.float32)
    assert float(gpu.argreduce(_dev(v), True).cpu().numpy()[0]) == O.argreduce(v, True) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("quantized", [False, True])
def test_embedding_col_matches_checker(quantized):
    """Column gather from a [dim, vocab] head (the reference's EmbeddingCol.cu): fp16 matrix, and int8 values
    with one fp16 scale per 32 rows and column; bit-exact against the checker, strides padded to 4."""
    import torch

    from cut_b200 import ops
    from oracle import oracle as O

    rng = np.random.default_rng(12)
    dim, vocab = 96, 37
    vstride = (vocab + 3) // 4 * 4
    idx = np.array([0, 36, 5, 5, 17], dtype=np.uint32)
    if quantized:
        m = np.zeros((dim, vstride), dtype=np.int8)
        m[:, :vocab] = rng.integers(-128, 128, size=(dim, vocab), dtype=np.int16).astype(np.int8)
        sc = np.zeros((dim // 32, vstride), dtype=np.float16)
        sc[:, :vocab] = np.abs(rng.normal(0, 0.02, size=(dim // 32, vocab))).astype(np.float16)
        want = O.embedding_col(idx, m, sc.view(np.uint16))
        got = ops.embedding_col(torch.from_numpy(idx.astype(np.int32)).cuda(), torch.from_numpy(m).cuda(),
                                torch.from_numpy(sc).cuda(), vocab=vocab)
    else:
        m = np.zeros((dim, vstride), dtype=np.float16)
        m[:, :vocab] = rng.normal(0, 1, size=(dim, vocab)).astype(np.float16)
        want = O.embedding_col(idx, m.view(np.uint16))
        got = ops.embedding_col(torch.from_numpy(idx.astype(np.int32)).cuda(), torch.from_numpy(m).cuda(), vocab=vocab)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # an index past the vocabulary is reported and written as zeros, never read
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bad = torch.tensor([3, vocab], dtype=torch.int32, device="cuda")
    mt = torch.from_numpy(m).cuda()
    out = ops.embedding_col(bad, mt, torch.from_numpy(sc).cuda() if quantized else None, vocab=vocab, status=status)
    assert int(status.item()) == L.ERR_INVALID and bool((out[1] == 0).all())


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [synth.Q8_0, synth.Q4_0, synth.Q4_K, synth.Q6_K, synth.Q5_0])
def test_embedding_blocks_equals_dequantised_rows(fmt):
    """Row gather from a table kept as raw GGUF blocks: every gathered row has the float32 bits of the checker's
    dequantised row."""
    import torch

    from cut_b200 import ops
    from oracle import oracle as O

    rows, cols = 50, 512
    raw = synth.make_weights(fmt, rows, cols, seed=60 + fmt)
    table = O.dequant_rows(fmt, raw, rows, cols)
    idx = np.array([49, 0, 7, 7, 31], dtype=np.int32)
    got = ops.embedding_blocks(torch.from_numpy(idx).cuda(), torch.from_numpy(raw).cuda(), fmt, rows, cols)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), table[idx].view(np.uint32))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.embedding_blocks(torch.tensor([rows], dtype=torch.int32, device="cuda"), torch.from_numpy(raw).cuda(), fmt, rows, cols,
                               status=status)
    assert int(status.item()) == L.ERR_INVALID and bool((out == 0).all())


@pytest.mark.gpu
def test_copy_batch_moves_every_range():
    """cutb_copy_batch: n device-to-device byte ranges in one launch (sizes that are not multiples of 16, an empty
    range, a range larger than one block's stride), table in device memory."""
    import torch

    from cut_b200 import _lib as L

    rng = np.random.default_rng(8)
    sizes = [44032, 8192, 4, 0, 1000003, 17, 16]
    src = [torch.from_numpy(rng.integers(0, 256, max(s, 16), dtype=np.uint8)).cuda() for s in sizes]
    dst = [torch.full((max(s, 16) + 16,), 7, dtype=torch.uint8, device="cuda") for s in sizes]
    table = torch.tensor([[a.data_ptr(), b.data_ptr(), s] for a, b, s in zip(src, dst, sizes)], dtype=torch.int64, device="cuda")
    L.check(L.lib().cutb_copy_batch(table.data_ptr(), len(sizes), max(sizes), None))
    torch.cuda.synchronize()
    for a, b, s in zip(src, dst, sizes):
        assert torch.equal(b[:s], a[:s]) and bool((b[s:] == 7).all())
    assert L.lib().cutb_copy_batch(None, 3, 16, None) == L.ERR_INVALID
    assert L.lib().cutb_copy_batch(None, 0, 0, None) == L.OK
