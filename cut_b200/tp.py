"""Row-sharded tensor parallelism for the quantized matmul (one process per GPU).

Output rows (N) are independent, so rank r of g owns GGUF rows
[r * N / g, (r + 1) * N / g): one contiguous byte range of the tensor, which
never moves.  Activations are replicated; every rank computes its slice of C.
The slices meet either through one NCCL all-gather (`all_gather_rows`) or inside the
mat-vec kernel itself (`ScatterGroup`): its epilogue stores the slice into every rank's
full output through peer-mapped pointers over NVLink; once per step a small exchange kernel
publishes the stores (system-scope fence, one add on every rank's arrival counter) and waits,
bounded, until every rank has done the same.
The reference has no counterpart (its only multi-device mode is a layer split
with a host bounce, runtime/Runtime.cpp:267-284); the split follows the plan
of keeping N / g a multiple of the kernels' 16-row tile.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib as L
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


PEER_HANDLE_BYTES = 64


class _RawCuda:
    """A raw device allocation presented through __cuda_array_interface__, so that torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class ScatterGroup:
    """Per-rank state of the fused exchange: `slots` full outputs [M, N] and one arrival counter in
    one device buffer that every other rank maps into its address space (cutb_peer_buffer_*: CUDA
    IPC, opened with the local device current; no multicast object is created).

    Use: `launch(desc, peers(slot))` for every mat-vec of a step, then `exchange()` once;
    afterwards `out[slot]` holds every rank's slice.  The ranks must pass a step
    boundary of their own (e.g. `dist.barrier()`) before a slot is written again.
    `close()` unmaps the peers' buffers and frees the own one (collective: every rank calls it).
    """

    def __init__(self, M: int, N: int, slots: int, device: torch.device, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 2 <= self.world <= L.MAX_PEERS:
            raise ValueError(f"ScatterGroup needs 2..{L.MAX_PEERS} ranks, got {self.world}")
        self.M, self.N, self.slots = M, N, slots
        self.device = device
        self.lo, self.hi = shard_rows(N, self.rank, self.world)
        # one allocation per rank: outputs first, the counter behind them on a 256-byte boundary
        out_bytes = (slots * M * N * 4 + 255) // 256 * 256
        self._bytes = out_bytes + 256
        lib = L.lib()
        own = C.c_void_p()
        handle = C.create_string_buffer(PEER_HANDLE_BYTES)
        with torch.cuda.device(device):
            L.check(lib.cutb_peer_buffer_alloc(self._bytes, C.byref(own), handle))
        self._own = own.value
        self.buf = torch.as_tensor(_RawCuda(self._own, self._bytes), device=device)
        self.out = self.buf[: slots * M * N * 4].view(torch.float32).view(slots, M, N)
        self.flag = self.buf[out_bytes: out_bytes + 8].view(torch.int64)
        handles = [None] * self.world
        dist.all_gather_object(handles, (device.index, handle.raw), group=group)
        self._opened = []
        self.peer_base = []
        for r, (owner_dev, raw) in enumerate(handles):
            if r == self.rank:
                self.peer_base.append(self._own)
                continue
            if not torch.cuda.can_device_access_peer(device.index, owner_dev):
                raise RuntimeError(f"GPU {device.index} cannot access GPU {owner_dev} as a peer")
            p = C.c_void_p()
            with torch.cuda.device(device):
                L.check(lib.cutb_peer_buffer_open(raw, C.byref(p)))
            self._opened.append(p.value)
            self.peer_base.append(p.value)
        torch.cuda.synchronize(device)
        self._flag_off = out_bytes
        self.steps = torch.zeros(1, dtype=torch.int64, device=device)  # waits made so far (device side)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._any_peers = self.peers(0)
        dist.barrier(group=group)

    def close(self) -> None:
        """Unmaps the peers' buffers, then (after every rank has done so) frees the own buffer."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        lib = L.lib()
        with torch.cuda.device(self.device):
            for p in self._opened:
                L.check(lib.cutb_peer_buffer_close(p))
        self._opened = []
        dist.barrier(group=self.group)  # nobody maps this rank's buffer any more
        self.out = self.flag = self.buf = None
        with torch.cuda.device(self.device):
            L.check(lib.cutb_peer_buffer_free(self._own))
        self._own = None

    def peers(self, slot: int) -> "L.PeerScatter":
        ps = L.PeerScatter()
        ps.world, ps.rank, ps.ldc_total, ps.n_offset = self.world, self.rank, self.N, self.lo
        for r in range(self.world):
            ps.C_peers[r] = self.peer_base[r] + slot * self.M * self.N * 4
            ps.flag_peers[r] = self.peer_base[r] + self._flag_off
        return ps

    def launch(self, desc, peers, stream_ptr: int) -> None:
        """One row-shard mat-vec whose epilogue stores its slice into `peers` (from `peers(slot)`)."""
        L.check(L.lib().cutb_qmatmul_scatter(C.byref(desc), C.byref(peers), stream_ptr))

    def exchange(self, stream_ptr: int) -> None:
        """Step boundary: publishes this rank's stores of the step and orders the stream behind every
        rank's (bounded).  The step count lives on the device, so the launch can be captured once
        and replayed."""
        L.check(L.lib().cutb_peer_exchange(C.byref(self._any_peers), self.steps.data_ptr(), self.status.data_ptr(), stream_ptr))
