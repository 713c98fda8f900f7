"""The plane-layout kernels against the reference's OWN CUDA kernels run on this GPU (cubins compiled from the
reference tree by oracle/build_ref_cuda.py, as its backend compiles them): same operands in the reference's
run-time layout, outputs within fp32 summation-order noise of each other, and both within 1e-5 of the CPU checker.
Skipped where the cubins were not built (no reference tree and no prebuilt files)."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import ref_cuda

pytestmark = pytest.mark.gpu


def _operands(q4, M, K, N, seed):
    rng = np.random.default_rng(seed)
    ldb = (N // 2 if q4 else N)
    B = rng.integers(0, 256, size=(K, ldb), dtype=np.uint8)
    S = rng.uniform(0.002, 0.02, size=(K // 32, N)).astype(np.float16)
    A = rng.normal(0, 1, (M, K)).astype(np.float32)
    return A, B, S


@pytest.mark.parametrize("q4,kernel", [(True, "MatMulQ4GemvKPar8"), (False, "MatMulQ8GemvKPar8")])
@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (1, 4096, 11008), (3, 1024, 264), (1, 96, 8)])
def test_plane_matvec_against_the_reference_cuda_matvec(q4, kernel, M, K, N):
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops

    if not ref_cuda.have(kernel):
        pytest.skip("reference cubins not built")
    A, B, S = _operands(q4, M, K, N, K + N + M)
    dA, dB, dS = (torch.from_numpy(x).cuda() for x in (A, B, S.view(np.uint16)))
    ldb = B.shape[1]
    ref_out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    ref_cuda.launch(kernel, dA, dB, dS, ref_out, M, K, N, stride_a=K, stride_b=ldb, stride_c=N, scale_stride=N)
    ours = ops.qmatmul(dA, dB, L.Q4_0 if q4 else L.Q8_0, N, layout=L.LAYOUT_KN_PLANES, scales=dS, ldb=ldb, lds=N,
                       variant=L.VARIANT_GEMV_PLANES)
    torch.cuda.synchronize()
    got, ref = ours.cpu().numpy().astype(np.float64), ref_out.cpu().numpy().astype(np.float64)
    want = O.qmatmul_planes(q4, False, A, B, S.view(np.uint16), M, K, N, acc64=True).astype(np.float64)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    assert rel(ref, want) <= 1e-5   # the reference's kernel is what the checker restates
    assert rel(got, want) <= 1e-5
    assert rel(got, ref) <= 1e-5


@pytest.mark.parametrize("q4,kernel", [(True, "MatMulQ4CoopMatTiled"), (False, "MatMulQ8CoopMatTiled")])
def test_block_gemm_against_the_reference_tensor_core_kernel(q4, kernel):
    """Prefill: the reference's tiled tensor-core kernel over planes against this library's GEMM over the same weights
    as GGUF blocks (planes built from the blocks by the device repacks).  Both round operands to fp16: 3e-3."""
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    if not ref_cuda.have(kernel):
        pytest.skip("reference cubins not built")
    M, K, N = 64, 1024, 256
    fmt = L.Q4_0 if q4 else L.Q8_0
    raw = torch.from_numpy(synth.make_weights(fmt, N, K, seed=77)).cuda()
    A = torch.from_numpy(synth.make_activations(M, K, 78, np.float32)).cuda()
    vals, scales = ops.separate_blocks(raw, fmt, N, K)
    if q4:
        planeB = ops.transpose_q4(vals, N, K)                      # [K, pad4(N / 2)]
    else:
        planeB = ops.transpose_2d(vals, ldo=(N + 3) // 4 * 4)     # [K, pad4(N)]
    planeS = ops.transpose_2d(scales, ldo=(N + 3) // 4 * 4)       # [K / 32, pad4(N)]
    ref_out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    ref_cuda.launch(kernel, A, planeB, planeS, ref_out, M, K, N, stride_a=K, stride_b=planeB.stride(0), stride_c=N,
                    scale_stride=planeS.stride(0))
    ours = ops.qmatmul(A, raw, fmt, N, variant=L.VARIANT_GEMM_TC)
    torch.cuda.synchronize()
    want = O.qmatmul_blocks(fmt, A.cpu().numpy(), raw.cpu().numpy(), M, K, N).astype(np.float64)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    assert rel(ref_out.cpu().numpy().astype(np.float64), want) <= 3e-3
    assert rel(ours.cpu().numpy().astype(np.float64), want) <= 3e-3


@pytest.mark.parametrize("q4,affine,kernel", [(True, False, "MatMulQ4CoopMatTiled"), (False, False, "MatMulQ8CoopMatTiled"), (True, True, None)])
@pytest.mark.parametrize("M,K,N", [(64, 1024, 256), (13, 4096, 5120), (200, 512, 1000)])
def test_plane_gemm_against_the_reference_tensor_core_kernel(q4, affine, kernel, M, K, N):
    """Prefill over the reference's [K, N] planes: the tcgen05 GEMM with plane converters (what CUTB_VARIANT_AUTO
    picks for this layout above four rows) against the reference's own tensor-core kernel on the same operands
    (where its tile shape takes them: N % 32 == 0) and against the CPU checker; fp16 operands on both sides: 3e-3."""
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops

    rng = np.random.default_rng(K + N + M)
    ldb, lds = ((N // 2 if q4 else N) + 3) // 4 * 4, (N + 3) // 4 * 4
    B = rng.integers(0, 256, size=(K, ldb), dtype=np.uint8)
    S = np.zeros((K // 32 * (2 if affine else 1), lds), np.float16)
    S[: K // 32] = rng.uniform(0.002, 0.02, size=(K // 32, lds)).astype(np.float16)
    if affine:
        S[K // 32:] = rng.uniform(-0.05, 0.05, size=(K // 32, lds)).astype(np.float16)
    A = rng.normal(0, 1, (M, K)).astype(np.float32)
    dA, dB, dS = (torch.from_numpy(x).cuda() for x in (A, B, S.view(np.uint16)))
    d, C_out, keep = ops.make_desc(dA, dB, L.Q4_0 if q4 else L.Q8_0, N, layout=L.LAYOUT_KN_PLANES, scales=dS, affine=affine, ldb=ldb, lds=lds)
    assert ops.select_variant(d) == L.VARIANT_GEMM_TC
    ours = ops.qmatmul(dA, dB, L.Q4_0 if q4 else L.Q8_0, N, layout=L.LAYOUT_KN_PLANES, scales=dS, affine=affine, ldb=ldb, lds=lds)
    torch.cuda.synchronize()
    want = O.qmatmul_planes(q4, affine, A, B, S.view(np.uint16), M, K, N, lda=K, ldb=ldb, lds=lds, acc64=True).astype(np.float64)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    assert rel(ours.cpu().numpy().astype(np.float64), want) <= 3e-3
    if kernel and N % 32 == 0 and ref_cuda.have(kernel):
        ref_out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
        ref_cuda.launch(kernel, dA, dB, dS, ref_out, M, K, N, stride_a=K, stride_b=ldb, stride_c=N, scale_stride=lds)
        torch.cuda.synchronize()
        assert rel(ref_out.cpu().numpy().astype(np.float64), want) <= 3e-3
        assert rel(ours.cpu().numpy().astype(np.float64), ref_out.cpu().numpy().astype(np.float64)) <= 1e-3


def _rope_tables(max_seq, hd):
    half = hd // 2
    freq = (np.float32(1.0) / np.power(np.float32(10000.0), (2 * np.arange(half, dtype=np.float32)) / np.float32(hd)))
    ang = np.arange(max_seq, dtype=np.float32)[:, None] * freq.astype(np.float32)[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


@pytest.mark.parametrize("kv", [np.float32, np.float16])
@pytest.mark.parametrize("n_heads,n_kv,hd,max_seq,seq", [(32, 8, 128, 2048, 515), (32, 8, 128, 2048, 2048), (4, 2, 8, 16, 7), (6, 3, 66, 64, 40),
                                                         (8, 8, 64, 256, 1)])
def test_attention_against_the_reference_cuda_kernel(kv, n_heads, n_kv, hd, max_seq, seq):
    """cutb_attention_decode (cluster or general kernel, whichever the shape selects) against the reference's own
    Attention.cu on the same caches; both within the usual tolerance of the float64 checker."""
    import torch

    from cut_b200 import ops

    name = "Attention_f16" if kv == np.float16 else "Attention"
    if not ref_cuda.have(name):
        pytest.skip("reference cubins not built")
    rng = np.random.default_rng(seq + hd)
    kv_dim = n_kv * hd
    ld = (kv_dim + 3) // 4 * 4
    q = rng.normal(0, 1, n_heads * hd).astype(np.float32)
    kc = rng.normal(0, 1, (max_seq, ld)).astype(kv)
    vc = rng.normal(0, 1, (max_seq, ld)).astype(kv)
    dq, dkc, dvc = (torch.from_numpy(x).cuda() for x in (q, kc, vc))
    params = torch.tensor([seq - 1, seq], dtype=torch.int32, device="cuda")
    scale = 1.0 / float(np.sqrt(np.float32(hd)))
    ref_out = torch.zeros(n_heads * hd, dtype=torch.float32, device="cuda")
    ref_cuda.attention(kv == np.float16, dq, dkc, dvc, params, ref_out, n_heads, n_kv, hd, scale)
    ws = ops.attention_workspace(n_heads, n_kv, hd, max_seq, "cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.attention_decode(dq, dkc, dvc, params, n_heads, n_kv, hd, ws, scale=scale, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = O.attention(q, kc, vc, seq, n_heads, n_kv, hd)
    g, r = got.cpu().numpy(), ref_out.cpu().numpy()
    assert np.all(np.abs(r - want) <= 1e-5 + 1e-4 * np.abs(want))   # the reference's kernel is what the checker restates
    assert np.all(np.abs(g - want) <= 1e-5 + 1e-4 * np.abs(want))
    assert np.all(np.abs(g - r) <= 2e-5 + 2e-4 * np.abs(r))


@pytest.mark.parametrize("kv", [np.float32, np.float16])
@pytest.mark.parametrize("n_heads,n_kv,hd,max_seq,pos", [(32, 8, 128, 600, 511), (4, 2, 8, 16, 0), (6, 3, 66, 64, 9)])
def test_rope_cache_write_against_the_reference_cuda_kernel(kv, n_heads, n_kv, hd, max_seq, pos):
    """cutb_rope_kv_write against the reference's FusedRoPEKVWrite.cu: the rotated query and the cache rows.  This
    library rounds the two products of a rotation separately (what the CPU checker and plain C give); NVRTC contracts
    the reference's `a * cos - b * sin` into a fused multiply-add, so the two differ by an ulp now and then."""
    import torch

    from cut_b200 import ops

    name = "FusedRoPEKVWrite_f16" if kv == np.float16 else "FusedRoPEKVWrite"
    if not ref_cuda.have(name):
        pytest.skip("reference cubins not built")
    rng = np.random.default_rng(pos + hd)
    q_dim, kv_dim = n_heads * hd, n_kv * hd
    ld = (kv_dim + 3) // 4 * 4
    cos_t, sin_t = _rope_tables(max_seq, hd)
    q, k, v = (rng.normal(0, 1, n).astype(np.float32) for n in (q_dim, kv_dim, kv_dim))
    kc0, vc0 = rng.normal(0, 1, (max_seq, ld)).astype(kv), rng.normal(0, 1, (max_seq, ld)).astype(kv)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    params = torch.tensor([pos, pos + 1], dtype=torch.int32, device="cuda")
    r_kc, r_vc, r_q = dev(kc0), dev(vc0), torch.zeros(q_dim, dtype=torch.float32, device="cuda")
    ref_cuda.rope_kv_write(kv == np.float16, dev(q), dev(k), dev(v), params, dev(cos_t), dev(sin_t), r_kc, r_vc, r_q, q_dim, kv_dim, hd)
    o_kc, o_vc = dev(kc0), dev(vc0)
    o_q = ops.rope_kv_write(dev(q), dev(k), dev(v), params, dev(cos_t), dev(sin_t), o_kc, o_vc, hd)
    torch.cuda.synchronize()
    assert np.allclose(o_q.cpu().numpy(), r_q.cpu().numpy(), rtol=1e-6, atol=1e-6)
    tol = dict(rtol=2e-3, atol=2e-3) if kv == np.float16 else dict(rtol=1e-6, atol=1e-6)
    assert np.allclose(o_kc.float().cpu().numpy(), r_kc.float().cpu().numpy(), **tol)
    assert torch.equal(o_vc, r_vc)                                    # v is stored as it is: identical
    other = np.arange(max_seq) != pos
    assert np.array_equal(o_kc.cpu().numpy()[other], kc0[other])      # only row pos is touched


def test_q4k_dequant_against_the_reference_cuda_kernel():
    """cutb_dequant (Q4_K) against the reference's DequantQ4K.cu, bit for bit."""
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    if not ref_cuda.have("DequantQ4K"):
        pytest.skip("reference cubins not built")
    rows, cols = 37, 1024
    raw = torch.from_numpy(synth.make_weights(synth.Q4_K, rows, cols, seed=12)).cuda()
    ref_out = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    ref_cuda.dequant_q4k(raw, ref_out, rows, cols)
    ours = ops.dequantize(raw, L.Q4_K, rows, cols)
    torch.cuda.synchronize()
    assert np.array_equal(ours.cpu().numpy().view(np.uint32), ref_out.cpu().numpy().view(np.uint32))


@pytest.mark.parametrize("name,fmt_attr,rows,cols", [("DequantQ5K", "Q5_K", 9, 1024), ("DequantQ6K", "Q6_K", 11, 768), ("DequantBF16", "BF16", 5, 520)])
def test_other_dequant_formats_against_the_reference_cuda_kernels(name, fmt_attr, rows, cols):
    """cutb_dequant for the rest of the reference's DequantFormat set against its own kernels, bit for bit (finite
    weights: the synthetic BF16 values contain no NaNs here)."""
    import torch

    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    if not ref_cuda.have(name):
        pytest.skip("reference cubins not built")
    fmt = getattr(L, fmt_attr)
    raw = torch.from_numpy(synth.make_weights(getattr(synth, fmt_attr), rows, cols, seed=21)).cuda()
    ref_out = torch.zeros((rows, (cols + 3) // 4 * 4), dtype=torch.float32, device="cuda")
    ref_cuda.dequant(name, raw, ref_out, rows, cols)
    ours = ops.dequantize(raw, fmt, rows, cols)
    torch.cuda.synchronize()
    a, b = ours.cpu().numpy(), ref_out.cpu().numpy()[:, :cols]
    finite = np.isfinite(b)
    assert finite.mean() > 0.99
    assert np.array_equal(a.view(np.uint32)[finite], b.view(np.uint32)[finite])


@pytest.mark.parametrize("rows,dim", [(1, 4096), (13, 5120), (3, 66)])
def test_rmsnorm_against_the_reference_cuda_kernel(rows, dim):
    import torch

    from cut_b200 import ops

    if not ref_cuda.have("RMSNorm"):
        pytest.skip("reference cubins not built")
    rng = np.random.default_rng(dim)
    ld = (dim + 3) // 4 * 4
    x = np.zeros((rows, ld), np.float32)
    x[:, :dim] = rng.normal(0, 2, (rows, dim))
    w = rng.uniform(0.5, 1.5, dim).astype(np.float32)
    dx, dw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    ref_out = torch.zeros_like(dx)
    ref_cuda.rmsnorm(dx, dw, ref_out, rows, dim, 1e-5)
    ours = ops.rmsnorm(dx[:, :dim] if ld == dim else dx[:, :dim], dw, 1e-5) if ld == dim else None
    if ours is None:  # a padded row stride: through the C ABI with the stride
        from cut_b200 import _lib as L

        ours = torch.zeros_like(dx)
        L.check(L.lib().cutb_rmsnorm(L.F32, dx.data_ptr(), dw.data_ptr(), ours.data_ptr(), rows, dim, ld, 1e-5, None))
    torch.cuda.synchronize()
    want = np.stack([O.rmsnorm(x[r, :dim], w, 1e-5) for r in range(rows)])
    assert np.allclose(ref_out.cpu().numpy()[:, :dim], want, rtol=2e-6, atol=1e-6)
    assert np.allclose(ours.cpu().numpy()[:, :dim], ref_out.cpu().numpy()[:, :dim], rtol=2e-6, atol=1e-6)


@pytest.mark.parametrize("n", [32000, 257, 5])
def test_argmax_against_the_reference_cuda_kernel_ties_included(n):
    """The reference's arg-max prefers, among equal maxima, the one its 256-thread scan and tree meet first; this
    library's kernel reproduces that rule in closed form.  Same index on data full of ties."""
    import torch

    from cut_b200 import ops

    if not ref_cuda.have("ReduceArgmax"):
        pytest.skip("reference cubins not built")
    rng = np.random.default_rng(n)
    for trial in range(4):
        v = rng.integers(0, 6 if trial else 1000, n).astype(np.float32)  # few distinct values: many ties
        dv = torch.from_numpy(v).cuda()
        ref_out = torch.zeros(1, dtype=torch.float32, device="cuda")
        ref_cuda.argmax(dv, ref_out, n)
        ours = ops.argreduce(dv, True)
        torch.cuda.synchronize()
        assert float(ours.item()) == float(ref_out.item()) and v[int(ours.item())] == v.max()


@pytest.mark.parametrize("kv", [np.float32, np.float16])
@pytest.mark.parametrize("n_heads,n_kv,hd,max_seq,T,start", [(32, 8, 128, 600, 40, 470), (4, 2, 8, 16, 5, 3), (6, 3, 66, 64, 20, 7)])
def test_batched_prefill_operators_against_the_reference_cuda_kernels(kv, n_heads, n_kv, hd, max_seq, T, start):
    """cutb_batched_kv_write and cutb_batched_attention against the reference's BatchedKVCacheWrite.cu and
    BatchedAttentionReadCache.cu, q / k / v as columns of one fused QKV matrix."""
    import torch

    from cut_b200 import ops

    if not ref_cuda.have("BatchedAttentionReadCache_f16" if kv == np.float16 else "BatchedAttentionReadCache"):
        pytest.skip("reference cubins not built")
    rng = np.random.default_rng(T + hd)
    q_dim, kv_dim = n_heads * hd, n_kv * hd
    width = q_dim + 2 * kv_dim
    ld = (kv_dim + 3) // 4 * 4
    cos_t, sin_t = _rope_tables(max_seq, hd)
    qkv = rng.normal(0, 1, (T, width)).astype(np.float32)
    kc0, vc0 = rng.normal(0, 1, (max_seq, ld)).astype(kv), rng.normal(0, 1, (max_seq, ld)).astype(kv)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    dq, dcos, dsin = dev(qkv), dev(cos_t), dev(sin_t)
    pos = dev(np.arange(start, start + T, dtype=np.int32))
    half = kv == np.float16
    r_kc, r_vc = dev(kc0), dev(vc0)
    ref_cuda.batched_kv_write(half, dq, dq, r_kc, r_vc, pos, dcos, dsin, T, kv_dim, hd, width, width, q_dim, q_dim + kv_dim)
    r_out = torch.zeros((T, q_dim), dtype=torch.float32, device="cuda")
    scale = 1.0 / float(np.sqrt(np.float32(hd)))
    ref_cuda.batched_attention(half, dq, r_kc, r_vc, pos, dcos, dsin, r_out, T, n_heads, n_kv, hd, scale, width, 0)
    o_kc, o_vc = dev(kc0), dev(vc0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.batched_kv_write(dq[:, q_dim:q_dim + kv_dim], dq[:, q_dim + kv_dim:], pos, dcos, dsin, o_kc, o_vc, hd, status=status)
    o_out = ops.batched_attention(dq[:, :q_dim], o_kc, o_vc, pos, dcos, dsin, n_heads, n_kv, hd, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    tol = dict(rtol=2e-3, atol=2e-3) if half else dict(rtol=1e-6, atol=1e-6)
    assert np.allclose(o_kc.float().cpu().numpy(), r_kc.float().cpu().numpy(), **tol)
    assert torch.equal(o_vc, r_vc)
    g, r = o_out.cpu().numpy(), r_out.cpu().numpy()
    assert np.all(np.abs(g - r) <= (2e-3 if half else 2e-5) + 2e-4 * np.abs(r))
