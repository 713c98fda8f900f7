"""GPU test of cutb_qmatmul_decode_noalloc, the decode mat-vec for embedders that
cannot allocate device memory (the whole GPU belongs to their own arena, or their
budget is fixed at start-up): its split-K scratch is an array built into the
library.  The output must equal the regular entry point's, call after call, and
shapes whose partial sums exceed the built-in array must be refused.  Collected
last on purpose, so a failure here cannot hide another test's result."""
import ctypes as C

import numpy as np
import pytest

from cut_b200 import _lib as L
from cut_b200 import synth

pytestmark = pytest.mark.gpu


def _desc(A, W, fmt, N, C_out):
    from cut_b200 import ops

    d, _, keep = ops.make_desc(A, W, fmt, N, C_out=C_out)
    return d, keep


@pytest.mark.parametrize("fmt", [synth.Q4_0, synth.Q8_0, synth.Q4_K])
def test_noalloc_matches_regular_entry_point_twice(fmt):
    import torch

    from cut_b200 import ops
    from gpu_util import dev, rel_l2

    assert torch.cuda.is_available()
    M, K, N = 8, 28672, 1024  # a 70B-shape shard: K is split across CTAs, partial sums need scratch
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        A = dev(synth.make_activations(M, K, 40 + call, np.float16))
        W = dev(synth.make_weights(fmt, N, K, seed=50 + call + fmt))
        want = ops.qmatmul(A, W, fmt, N)  # regular entry point, workspace from torch
        got = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        d, keep = _desc(A, W, fmt, N, got)
        assert ops.workspace_bytes(d) > 0  # the shape really uses scratch
        d.workspace, d.workspace_bytes = None, 0  # ignored by the no-alloc entry point
        L.check(L.lib().cutb_qmatmul_decode_noalloc(C.byref(d), stream))
        torch.cuda.synchronize()
        assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= 1e-3
        assert torch.equal(got, want)  # same kernels, same summation order


def test_noalloc_also_serves_shapes_without_scratch():
    import torch

    from cut_b200 import ops
    from gpu_util import dev

    A = dev(synth.make_activations(1, 4096, 3, np.float16))
    W = dev(synth.make_weights(synth.Q4_0, 2368, 4096, seed=4))
    want = ops.qmatmul(A, W, synth.Q4_0, 2368)
    got = torch.empty_like(want)
    d, keep = _desc(A, W, synth.Q4_0, 2368, got)
    L.check(L.lib().cutb_qmatmul_decode_noalloc(C.byref(d), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_noalloc_rejects_what_it_cannot_hold():
    import torch

    from gpu_util import dev

    lib = L.lib()
    stream = torch.cuda.current_stream().cuda_stream
    # partial sums of this shape (ksplit * 16 * 8192 floats) exceed the 4 MiB array
    M, K, N = 16, 28672, 8192
    A = torch.zeros((M, K), dtype=torch.float16, device="cuda")
    W = torch.zeros(N * synth.row_bytes(synth.Q4_0, K), dtype=torch.uint8, device="cuda")
    out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    d, keep = _desc(A, W, synth.Q4_0, N, out)
    from cut_b200 import ops

    assert ops.workspace_bytes(d) > 4 << 20  # the precondition of this case: the shape needs more than the array holds
    assert lib.cutb_qmatmul_decode_noalloc(C.byref(d), stream) == L.ERR_WORKSPACE
    assert b"built-in array" in lib.cutb_last_error()
    # prefill-sized batches are not decode mat-vecs
    A2 = dev(synth.make_activations(64, 256, 1, np.float16))
    W2 = dev(synth.make_weights(synth.Q4_0, 16, 256, seed=2))
    out2 = torch.zeros((64, 16), dtype=torch.float32, device="cuda")
    d2, keep2 = _desc(A2, W2, synth.Q4_0, 16, out2)
    assert lib.cutb_qmatmul_decode_noalloc(C.byref(d2), stream) == L.ERR_UNSUPPORTED
    assert lib.cutb_qmatmul_decode_noalloc(None, stream) == L.ERR_INVALID


def test_noalloc_rejects_flag_combinations_the_kernel_cannot_run():
    """The flag guards of cutb_qmatmul hold for this entry point too: paired gate/up rows on a shape that
    splits K, and a fused RMSNorm without its weight, are refused before anything is launched."""
    import torch

    from cut_b200 import ops

    lib = L.lib()
    stream = torch.cuda.current_stream().cuda_stream
    M, K, N = 1, 28672, 1024  # splits K
    A = torch.zeros((M, K), dtype=torch.float16, device="cuda")
    W = torch.zeros(N * synth.row_bytes(synth.Q4_0, K), dtype=torch.uint8, device="cuda")
    out = torch.full((M, N), 7.0, dtype=torch.float32, device="cuda")
    d, keep = _desc(A, W, synth.Q4_0, N, out)
    assert ops.workspace_bytes(d) > 0
    d.flags = L.FLAG_GLU_PAIRS
    d.fusion_type, d.fusion_op = L.FUSION_UNARY, 133
    assert lib.cutb_qmatmul_decode_noalloc(C.byref(d), stream) == L.ERR_UNSUPPORTED
    assert b"paired gate/up" in lib.cutb_last_error()
    d.flags = L.FLAG_A_RMSNORM  # a_norm_weight stays null
    d.fusion_type, d.fusion_op = 0, 0
    assert lib.cutb_qmatmul_decode_noalloc(C.byref(d), stream) == L.ERR_INVALID
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())  # nothing ran
