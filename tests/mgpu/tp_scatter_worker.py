"""One rank of the fused row-shard exchange test (launched by torchrun from test_gpu_tp_scatter.py).

Every rank owns an equal slice of the weight rows, runs the mat-vec whose epilogue scatters the slice
into every rank's full output, waits on its arrival counter and checks the assembled output against
(a) the plain single-GPU kernel run on every slice, bit for bit, and (b) the CPU checker.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from cut_b200 import _lib as L  # noqa: E402
from cut_b200 import ops, synth, tp  # noqa: E402
from oracle import oracle as O  # noqa: E402  (checker)


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.current_stream().cuda_stream
    failures = []
    # 4096 rows per rank: whole K per CTA, the mat-vec kernel scatters; 512 rows per rank: K is
    # split and the reduction kernel scatters
    for fmt, M, adt, rows_per_rank in ((L.Q4_0, 1, np.float16, 4096), (L.Q4_K, 2, np.float16, 4096),
                                       (L.Q8_0, 1, np.float32, 2048), (L.Q4_0, 1, np.float16, 512)):
        K, N = 4096, rows_per_rank * world
        Wfull = synth.make_weights(fmt, N, K, seed=5)  # same on every rank
        A_h = synth.make_activations(M, K, 9, adt)
        lo, hi = tp.shard_rows(N, rank, world)
        rb = synth.row_bytes(fmt, K)
        W_local = torch.from_numpy(Wfull[lo * rb: hi * rb].copy()).to(dev)
        A = torch.from_numpy(A_h).to(dev)
        grp = tp.ScatterGroup(M, N, slots=2, device=dev)
        c_dummy = torch.empty((M, hi - lo), dtype=torch.float32, device=dev)
        d, _, keep = ops.make_desc(A, W_local, fmt, hi - lo, C_out=c_dummy, status=grp.status, variant=L.VARIANT_GEMV_MMA)
        need = ops.workspace_bytes(d)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        if need:
            d.workspace, d.workspace_bytes = ws.data_ptr(), need
        # every rank's slice on this GPU through the plain entry point (same shape, hence the same
        # launch plan and summation order as the rank that owns the slice)
        ref_dev = np.concatenate(
            [ops.qmatmul(A, torch.from_numpy(Wfull[a * rb: b * rb].copy()).to(dev), fmt, b - a).cpu().numpy()
             for a, b in (tp.shard_rows(N, r, world) for r in range(world))], axis=1)
        ref_cpu = O.qmatmul_blocks(fmt, A_h.astype(np.float32), Wfull, M, K, N)
        for step in range(3):
            slot = step & 1
            grp.out[slot].zero_()
            torch.cuda.synchronize()
            dist.barrier()  # step boundary: nobody still reads or clears the slot
            grp.launch(d, grp.peers(slot), stream)
            grp.exchange(stream)
            torch.cuda.synchronize()
            got = grp.out[slot].cpu().numpy()
            if int(grp.status.item()) != 0:
                failures.append(f"fmt {fmt} step {step}: status {int(grp.status.item())}")
            if not np.array_equal(got, ref_dev):
                bad = int(np.sum(got != ref_dev))
                failures.append(f"fmt {fmt} step {step}: {bad} of {got.size} values differ from the single-GPU kernel")
            rel = float(np.linalg.norm(got - ref_cpu) / np.linalg.norm(ref_cpu))
            if not rel <= 1e-3:
                failures.append(f"fmt {fmt} step {step}: rel-L2 {rel} against the checker")
        dist.barrier()
        grp.close()
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    if failures:
        print(f"rank {rank}: " + "; ".join(failures), flush=True)
    if rank == 0:
        print("TP_SCATTER_OK" if int(flag.item()) == 0 else "TP_SCATTER_FAILED", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    code = 0 if int(flag.item()) == 0 else 1
    dist.destroy_process_group()
    return code


if __name__ == "__main__":
    sys.exit(main())
