"""Row-sharded tensor parallelism for the quantized matmul (one process per GPU).

Output rows (N) are independent, so rank r of g owns GGUF rows
[r * N / g, (r + 1) * N / g): one contiguous byte range of the tensor, which
never moves.  Activations are replicated; every rank computes its slice of C
and one all-gather over NCCL (NVLink / NVSwitch) assembles the full output.
The reference has no counterpart (its only multi-device mode is a layer split
with a host bounce, runtime/Runtime.cpp:267-284); the split follows the plan
of keeping N / g a multiple of the kernels' 16-row tile.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import synth

ROW_TILE = 16


def shard_rows(N: int, rank: int, world: int) -> tuple[int, int]:
    """Row range [lo, hi) of `rank`: equal shares rounded to the 16-row tile, remainder to the last ranks."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    tiles = (N + ROW_TILE - 1) // ROW_TILE
    lo_t = tiles * rank // world
    hi_t = tiles * (rank + 1) // world
    return min(lo_t * ROW_TILE, N), min(hi_t * ROW_TILE, N)


def shard_bytes(fmt: int, N: int, K: int, rank: int, world: int) -> tuple[int, int]:
    """Byte range of the rank's rows inside the raw GGUF tensor."""
    lo, hi = shard_rows(N, rank, world)
    rb = synth.row_bytes(fmt, K)
    return lo * rb, hi * rb


def all_gather_rows(c_local: torch.Tensor, N: int, group=None) -> torch.Tensor:
    """[M, rows_of_this_rank] slices -> [M, N] on every rank (uneven shares allowed)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    M = c_local.shape[0]
    sizes = [shard_rows(N, r, world) for r in range(world)]
    assert c_local.shape[1] == sizes[rank][1] - sizes[rank][0]
    width = max(hi - lo for lo, hi in sizes)
    send = c_local.new_zeros((M, width))
    send[:, : c_local.shape[1]] = c_local
    recv = c_local.new_empty((world * M, width))  # rank-major concatenation along dim 0
    dist.all_gather_into_tensor(recv, send, group=group)
    recv = recv.view(world, M, width)
    out = c_local.new_empty((M, N))
    for r, (lo, hi) in enumerate(sizes):
        out[:, lo:hi] = recv[r, :, : hi - lo]
    return out
