"""GPU parity of the decode-step attention operators against the CPU checker: fused RoPE + KV-cache
write bit-exact (fp32 and fp16 caches), attention within 1e-5 absolute + 1e-4 relative of the
float64 checker (the reference's own tests allow 1e-3, tests/runtime/RuntimeTests.cpp:6025-6030)."""
import numpy as np
import pytest

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


def rope_tables(max_seq, head_dim, theta=10000.0):
    # interface/runner/llama/llama.cpp:1652-1666
    half = head_dim // 2
    freq = (1.0 / np.power(np.float32(theta), (2 * np.arange(half, dtype=np.float32)) / np.float32(head_dim))).astype(np.float32)
    ang = np.arange(max_seq, dtype=np.float32)[:, None] * freq[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def reference_test_data(count, seed):
    """Uniform [0.1, 10) like the reference's generateTestData (values differ; the distribution is the same)."""
    return np.random.default_rng(seed).uniform(0.1, 10.0, count).astype(np.float32)


@pytest.mark.parametrize("kv", [np.float32, np.float16])
@pytest.mark.parametrize("n_heads,n_kv,hd,max_seq,pos", [(32, 8, 128, 2048, 0), (32, 8, 128, 2048, 777), (32, 8, 128, 2048, 2047),
                                                         (4, 2, 8, 16, 3), (1, 1, 4, 8, 2), (6, 3, 66, 40, 39)])
def test_rope_kv_write_bit_exact(gpu, kv, n_heads, n_kv, hd, max_seq, pos):
    import torch

    rng = np.random.default_rng(pos + hd)
    q = rng.uniform(-1, 1, n_heads * hd).astype(np.float32)
    k = rng.uniform(-1, 1, n_kv * hd).astype(np.float32)
    v = rng.uniform(-1, 1, n_kv * hd).astype(np.float32)
    ld = (n_kv * hd + 3) // 4 * 4
    cos_t, sin_t = rope_tables(max_seq, hd)
    kc = rng.uniform(-1, 1, (max_seq, ld)).astype(kv)
    vc = rng.uniform(-1, 1, (max_seq, ld)).astype(kv)
    kc_ref, vc_ref = kc.copy(), vc.copy()
    q_ref = O.rope_kv_write(q, k, v, pos, cos_t, sin_t, kc_ref, vc_ref, hd)
    params = _dev(np.array([pos, pos + 1], dtype=np.uint32).view(np.int32))
    dkc, dvc = _dev(kc), _dev(vc)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_out = gpu.rope_kv_write(_dev(q), _dev(k), _dev(v), params, _dev(cos_t), _dev(sin_t), dkc, dvc, hd, status=status)
    assert np.array_equal(q_out.cpu().numpy().view(np.uint32), q_ref.view(np.uint32))
    bits = np.uint16 if kv == np.float16 else np.uint32
    assert np.array_equal(dkc.cpu().numpy().view(bits), kc_ref.view(bits))  # row pos written, every other row untouched
    assert np.array_equal(dvc.cpu().numpy().view(bits), vc_ref.view(bits))
    assert int(status.item()) == 0


def test_rope_position_outside_cache_is_reported_not_written(gpu):
    import torch

    hd, n_kv, max_seq = 8, 2, 4
    kc = np.zeros((max_seq, n_kv * hd), np.float32)
    dkc, dvc = _dev(kc), _dev(kc)
    cos_t, sin_t = rope_tables(max_seq, hd)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = np.ones(n_kv * hd, np.float32)
    gpu.rope_kv_write(_dev(np.ones(4 * hd, np.float32)), _dev(x), _dev(x), _dev(np.array([max_seq, max_seq + 1], np.int32)), _dev(cos_t),
                      _dev(sin_t), dkc, dvc, hd, status=status)
    assert int(status.item()) == 1 and not dkc.cpu().numpy().any() and not dvc.cpu().numpy().any()


CASES = [
    # n_heads, n_kv, head_dim, max_seq, seq_len
    (1, 1, 4, 8, 3),          # the reference's SingleHeadBasic geometry
    (4, 2, 8, 16, 4),         # its MultiHeadGQA geometry
    (32, 8, 128, 2048, 1),
    (32, 8, 128, 2048, 5),
    (32, 8, 128, 2048, 513),
    (32, 8, 128, 2048, 2048),
    (32, 32, 64, 300, 299),   # no grouping, head_dim 64
    (8, 1, 96, 1000, 777),    # 8 query heads on one KV head, 12-element lanes
    (6, 3, 66, 40, 40),       # head_dim not a multiple of 32: scalar loads
    (16, 2, 128, 8192, 8000),  # 512-position slices
    (6, 2, 64, 500, 333),     # three query heads per KV head: general kernel with vector loads
]


@pytest.mark.parametrize("kv", [np.float32, np.float16])
@pytest.mark.parametrize("n_heads,n_kv,hd,max_seq,seq", CASES)
def test_attention_decode_matches_checker(gpu, kv, n_heads, n_kv, hd, max_seq, seq):
    import torch

    rng = np.random.default_rng(seq * 7 + hd)
    ld = (n_kv * hd + 3) // 4 * 4
    if max_seq <= 16:  # reference geometry: its uniform [0.1, 10) data (large, nearly one-hot softmax)
        q = reference_test_data(n_heads * hd, 42)
        kc = reference_test_data(max_seq * ld, 100).reshape(max_seq, ld).astype(kv)
        vc = reference_test_data(max_seq * ld, 200).reshape(max_seq, ld).astype(kv)
    else:
        q = rng.normal(0, 1.0, n_heads * hd).astype(np.float32)
        kc = rng.normal(0, 1.0, (max_seq, ld)).astype(kv)
        vc = rng.normal(0, 1.0, (max_seq, ld)).astype(kv)
    want = O.attention(q, kc, vc, seq, n_heads, n_kv, hd)
    ws = gpu.attention_workspace(n_heads, n_kv, hd, max_seq, "cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    params = _dev(np.array([seq - 1, seq], np.int32))
    dq, dk, dv = _dev(q), _dev(kc), _dev(vc)
    for _ in range(2):  # the second launch proves the arrival counters were left at zero
        got = gpu.attention_decode(dq, dk, dv, params, n_heads, n_kv, hd, ws, status=status).cpu().numpy()
        assert np.all(np.abs(got - want) <= 1e-5 + 1e-4 * np.abs(want)), float(np.max(np.abs(got - want)))
    assert int(status.item()) == 0
    assert not ws[:256].cpu().numpy().any()


@pytest.mark.parametrize("kv", [np.float32, np.float16])
@pytest.mark.parametrize("n_heads,n_kv,hd,max_seq,positions", [
    (32, 8, 128, 2048, [0, 1, 255, 256, 511, 2047]),  # cluster kernel; rows at slice boundaries (fp32 caches: two launches)
    (8, 8, 64, 64, [0, 7, 8, 63]),                     # cluster kernel, one query head per KV head
    (6, 2, 64, 100, [0, 50, 99]),                      # three heads per KV head: rotation kernel + general attention
    (4, 2, 8, 16, [0, 3, 15]),                         # tiny head_dim: scalar general kernel
])
def test_rope_attention_decode_equals_the_two_calls(gpu, kv, n_heads, n_kv, hd, max_seq, positions):
    import torch

    rng = np.random.default_rng(hd + max_seq)
    ld = (n_kv * hd + 3) // 4 * 4
    cos_t, sin_t = rope_tables(max_seq, hd)
    kc = rng.normal(0, 1, (max_seq, ld)).astype(kv)
    vc = rng.normal(0, 1, (max_seq, ld)).astype(kv)
    dkc, dvc = _dev(kc), _dev(vc)
    kc_ref, vc_ref = kc.copy(), vc.copy()
    ws = gpu.attention_workspace(n_heads, n_kv, hd, max_seq, "cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bits = np.uint16 if kv == np.float16 else np.uint32
    for pos in positions:
        q = rng.normal(0, 1, n_heads * hd).astype(np.float32)
        k = rng.normal(0, 1, n_kv * hd).astype(np.float32)
        v = rng.normal(0, 1, n_kv * hd).astype(np.float32)
        q_ref = O.rope_kv_write(q, k, v, pos, cos_t, sin_t, kc_ref, vc_ref, hd)
        want = O.attention(q_ref, kc_ref, vc_ref, pos + 1, n_heads, n_kv, hd)
        got = gpu.rope_attention_decode(_dev(q), _dev(k), _dev(v), _dev(np.array([pos, pos + 1], np.int32)), _dev(cos_t), _dev(sin_t),
                                        dkc, dvc, n_heads, n_kv, hd, ws, status=status).cpu().numpy()
        assert np.all(np.abs(got - want) <= 1e-5 + 1e-4 * np.abs(want)), (pos, float(np.max(np.abs(got - want))))
        assert np.array_equal(dkc.cpu().numpy().view(bits), kc_ref.view(bits))  # row pos written bit-exactly, nothing else touched
        assert np.array_equal(dvc.cpu().numpy().view(bits), vc_ref.view(bits))
    assert int(status.item()) == 0
    # a position past the cache: reported, nothing written
    before = dkc.clone()
    gpu.rope_attention_decode(_dev(q), _dev(k), _dev(v), _dev(np.array([max_seq, max_seq], np.int32)), _dev(cos_t), _dev(sin_t), dkc, dvc,
                              n_heads, n_kv, hd, ws, status=status)
    assert int(status.item()) == 1 and torch.equal(before, dkc)


@pytest.mark.parametrize("kv", [np.float32, np.float16])
@pytest.mark.parametrize("n_heads,n_kv,hd,max_seq,T,start", [(32, 8, 128, 600, 512, 0), (4, 2, 8, 16, 5, 3), (6, 3, 66, 64, 20, 7),
                                                              (8, 2, 64, 1400, 700, 650), (4, 4, 32, 2100, 90, 1990),
                                                              (8, 4, 128, 300, 77, 101),   # a ragged last tile of tokens and of rows
                                                              (4, 1, 64, 128, 16, 0)])     # the smallest batch the tensor-core kernel takes
def test_batched_prefill_operators_match_checker(gpu, kv, n_heads, n_kv, hd, max_seq, T, start):
    """cutb_batched_kv_write (bit-exact cache rows, inputs as columns of one fused QKV matrix) and
    cutb_batched_attention (every token over the rows up to its own) against the checker run token by token."""
    import torch

    rng = np.random.default_rng(T + hd)
    q_dim, kv_dim = n_heads * hd, n_kv * hd
    ld = (kv_dim + 3) // 4 * 4
    cos_t, sin_t = rope_tables(max_seq, hd)
    qkv = rng.normal(0, 1, (T, q_dim + 2 * kv_dim)).astype(np.float32)
    kc = rng.normal(0, 1, (max_seq, ld)).astype(kv)
    vc = rng.normal(0, 1, (max_seq, ld)).astype(kv)
    kc_ref, vc_ref = kc.copy(), vc.copy()
    want = np.zeros((T, q_dim), np.float32)
    # the float64 checker is slow on long ranges: a few tokens, the chunk borders of the 512-row walk among them
    sel = np.arange(T) if T <= 24 else np.array([i for i in (0, 1, 100, 255, 256, 511, 512 - start, 1023 - start, 1024 - start, T - 1)
                                                 if 0 <= i < T])
    q_ref = {}
    for i in range(T):
        q_ref[i] = O.rope_kv_write(qkv[i, :q_dim], qkv[i, q_dim:q_dim + kv_dim], qkv[i, q_dim + kv_dim:], start + i, cos_t, sin_t,
                                   kc_ref, vc_ref, hd)
    for i in sel:
        want[i] = O.attention(q_ref[int(i)], kc_ref, vc_ref, start + int(i) + 1, n_heads, n_kv, hd)
    dq, dkc, dvc = _dev(qkv), _dev(kc), _dev(vc)
    pos = _dev(np.arange(start, start + T, dtype=np.int32))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gpu.batched_kv_write(dq[:, q_dim:q_dim + kv_dim], dq[:, q_dim + kv_dim:], pos, _dev(cos_t), _dev(sin_t), dkc, dvc, hd, status=status)
    bits = np.uint16 if kv == np.float16 else np.uint32
    assert np.array_equal(dkc.cpu().numpy().view(bits), kc_ref.view(bits))
    assert np.array_equal(dvc.cpu().numpy().view(bits), vc_ref.view(bits))
    got = gpu.batched_attention(dq[:, :q_dim], dkc, dvc, pos, _dev(cos_t), _dev(sin_t), n_heads, n_kv, hd, status=status).cpu().numpy()
    assert int(status.item()) == 0
    if kv == np.float16 and hd in (64, 128) and T >= 16:
        # the tensor-core kernel: rotated queries and probabilities rounded to fp16 (the cache already is), fp32 sums
        assert np.all(np.abs(got[sel] - want[sel]) <= 2e-3 + 2e-3 * np.abs(want[sel]))
        assert np.linalg.norm(got[sel] - want[sel]) / np.linalg.norm(want[sel]) <= 1e-3
    else:
        assert np.all(np.abs(got[sel] - want[sel]) <= 1e-5 + 1e-4 * np.abs(want[sel]))


def test_batched_attention_range_limit_and_glu_pairs(gpu):
    import torch

    n_heads, n_kv, hd, max_seq = 2, 1, 32, 1024
    cos_t, sin_t = rope_tables(max_seq, hd)
    kc = torch.zeros((max_seq, hd), device="cuda")
    q = torch.zeros((1, n_heads * hd), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gpu.batched_attention(q, kc, kc, _dev(np.array([600], np.int32)), _dev(cos_t), _dev(sin_t), n_heads, n_kv, hd, status=status)
    assert int(status.item()) == 0  # rows past 511 are walked in further chunks
    gpu.batched_attention(q, kc, kc, _dev(np.array([1024], np.int32)), _dev(cos_t), _dev(sin_t), n_heads, n_kv, hd, status=status)
    assert int(status.item()) == 1  # a position past the cache is reported, never read
    x = np.random.default_rng(0).normal(0, 2, (7, 20)).astype(np.float32)
    got = gpu.glu_pairs(_dev(x)).cpu().numpy()
    want = np.array([[O.epilogue(float(x[r, 2 * i]), 1, 133) * np.float32(x[r, 2 * i + 1]) for i in range(10)] for r in range(7)], np.float32)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-7)


def test_attention_empty_cache_and_clamped_length(gpu):
    import torch

    n_heads, n_kv, hd, max_seq = 4, 2, 32, 64
    rng = np.random.default_rng(3)
    q = rng.normal(0, 1, n_heads * hd).astype(np.float32)
    kc = rng.normal(0, 1, (max_seq, n_kv * hd)).astype(np.float32)
    vc = rng.normal(0, 1, (max_seq, n_kv * hd)).astype(np.float32)
    ws = gpu.attention_workspace(n_heads, n_kv, hd, max_seq, "cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = gpu.attention_decode(_dev(q), _dev(kc), _dev(vc), _dev(np.array([0, 0], np.int32)), n_heads, n_kv, hd, ws, status=status)
    assert not out.cpu().numpy().any() and int(status.item()) == 0  # nothing cached: zeros, as the reference's empty sum
    out = gpu.attention_decode(_dev(q), _dev(kc), _dev(vc), _dev(np.array([99, 100], np.int32)), n_heads, n_kv, hd, ws, status=status)
    want = O.attention(q, kc, vc, max_seq, n_heads, n_kv, hd)
    assert int(status.item()) == 1  # seqLen past the cache: clamped to the cache and reported
    assert np.allclose(out.cpu().numpy(), want, rtol=1e-4, atol=1e-5)


def test_attention_argument_errors(gpu):
    import torch

    from cut_b200 import _lib as L

    q = torch.zeros(4 * 32, device="cuda")
    kc = torch.zeros((8, 64), device="cuda")
    params = torch.zeros(2, dtype=torch.int32, device="cuda")
    ws = gpu.attention_workspace(4, 2, 32, 8, "cuda")
    with pytest.raises(L.CutbError):
        gpu.attention_decode(q, kc, kc, params, 4, 3, 32, ws)       # heads not a multiple of KV heads
    with pytest.raises(L.CutbError):
        gpu.attention_decode(q, kc, kc, params, 4, 2, 32, ws[:64])  # workspace too small
    with pytest.raises(L.CutbError):
        gpu.rope_kv_write(q, kc[0], kc[0], params, q, q, kc, kc, 7)  # odd head_dim
