"""Host logic of the row-sharded multi-GPU path on CPU: two gloo ranks shard a
GGUF tensor by rows, each computes its slice with the CPU checker (standing in
for the kernel, which needs a GPU) and the all-gather reproduces the unsharded
result bit for bit."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, fmt, M, K, N, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from cut_b200 import synth, tp
    from oracle import oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    W = synth.make_weights(fmt, N, K, seed=5)
    A = synth.make_activations(M, K, 6)
    lo, hi = tp.shard_rows(N, rank, world)
    b0, b1 = tp.shard_bytes(fmt, N, K, rank, world)
    c_local = O.qmatmul_blocks(fmt, A, W[b0:b1], M, K, hi - lo)
    full = tp.all_gather_rows(torch.from_numpy(c_local), N)
    ref = O.qmatmul_blocks(fmt, A, W, M, K, N)
    ok = np.array_equal(full.numpy(), ref)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("fmt,N", [(1, 1000), (2, 48)])
def test_row_sharded_all_gather_two_ranks(tmp_path, fmt, N):
    world = 2
    port = 29500 + (os.getpid() + fmt) % 400
    mp.spawn(_worker, args=(world, port, fmt, 3, 256, N, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_shard_rows_cover_and_align():
    sys.path.insert(0, ROOT)
    from cut_b200 import tp

    for N in (16, 1000, 11008, 28672, 5):
        for world in (1, 2, 4, 8):
            ranges = [tp.shard_rows(N, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == N
            for (lo, hi), (lo2, _) in zip(ranges, ranges[1:]):
                assert hi == lo2 and lo % 16 == 0
    assert tp.shard_bytes(1, 11008, 4096, 1, 2) == (5504 * 2304, 11008 * 2304)
    with pytest.raises(ValueError):
        tp.shard_rows(16, 2, 2)
