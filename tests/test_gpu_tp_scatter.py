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
