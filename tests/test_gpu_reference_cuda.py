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
