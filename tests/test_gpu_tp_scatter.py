"""Fused row-shard exchange on two GPUs (skipped on a single-GPU box): the mat-vec's epilogue
stores its slice into both ranks' outputs through peer-mapped pointers; compared bit for bit with
the single-GPU kernel and within 1e-3 of the CPU checker.  Runs as torchrun child processes with
NVLS off; every device-side wait is bounded."""
import os
import socket
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.gpu
def test_scatter_epilogue_two_ranks():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "mgpu", "tp_scatter_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "TP_SCATTER_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]


@pytest.mark.gpu
def test_exchange_wait_runs_out_instead_of_hanging():
    """Failure detection of the fused exchange on one GPU: a two-rank exchange in which the other rank
    never signals.  The exchange kernel's wait is bounded (about a second): it must come back with
    CUTB_ERR_TIMEOUT in the status word and leave the stream and the context usable."""
    import ctypes as C
    import time

    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    sys.path.insert(0, ROOT)
    from cut_b200 import _lib as L

    dev = torch.device("cuda", 0)
    out = torch.zeros(16, dtype=torch.float32, device=dev)
    flags = torch.zeros(2 * 32, dtype=torch.int64, device=dev)  # two counters, 256 bytes apart
    steps = torch.zeros(1, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ps = L.PeerScatter()
    ps.world, ps.rank, ps.ldc_total, ps.n_offset = 2, 0, 16, 0
    for r in range(2):
        ps.C_peers[r] = out.data_ptr()
        ps.flag_peers[r] = flags.data_ptr() + 256 * r
    t0 = time.perf_counter()
    L.check(L.lib().cutb_peer_exchange(C.byref(ps), steps.data_ptr(), status.data_ptr(), None))
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(status.item()) == L.ERR_TIMEOUT
    assert 0.2 < waited < 10.0
    # this rank signalled both counters once, the missing rank never did; the step was counted
    assert flags[0].item() == 1 and flags[32].item() == 1 and steps.item() == 1
    # the context still works
    assert float((out + 1).sum().item()) == 16.0


@pytest.mark.gpu
def test_scatter_refuses_paired_rows_before_launching():
    """cutb_qmatmul_scatter shares the mat-vec's flag guards: paired gate/up rows cannot be scattered
    (the slice would go to desc->C and the peers would get nothing), so the call is refused and
    nothing is launched.  One GPU is enough: the refusal comes before any peer pointer is used."""
    import ctypes as C

    import numpy as np

    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    sys.path.insert(0, ROOT)
    from cut_b200 import _lib as L
    from cut_b200 import ops, synth

    dev = torch.device("cuda", 0)
    K, N = 4096, 256
    A = torch.from_numpy(synth.make_activations(1, K, 3, np.float16)).to(dev)
    W = torch.from_numpy(synth.make_weights(synth.Q4_0, N, K, seed=4)).to(dev)
    out = torch.full((1, 2 * N), 5.0, dtype=torch.float32, device=dev)
    flags = torch.zeros(64, dtype=torch.int64, device=dev)
    c_dummy = torch.zeros((1, N), dtype=torch.float32, device=dev)
    d, _, keep = ops.make_desc(A, W, synth.Q4_0, N, C_out=c_dummy, variant=L.VARIANT_GEMV_MMA)
    d.flags = L.FLAG_GLU_PAIRS
    d.fusion_type, d.fusion_op = L.FUSION_UNARY, 133
    ps = L.PeerScatter()
    ps.world, ps.rank, ps.ldc_total, ps.n_offset = 2, 0, 2 * N, 0
    for r in range(2):
        ps.C_peers[r] = out.data_ptr()
        ps.flag_peers[r] = flags.data_ptr() + 256 * r
    rc = L.lib().cutb_qmatmul_scatter(C.byref(d), C.byref(ps), None)
    assert rc == L.ERR_UNSUPPORTED and b"paired gate/up" in L.lib().cutb_last_error()
    torch.cuda.synchronize()
    assert bool((out == 5.0).all()) and bool((c_dummy == 0).all())
