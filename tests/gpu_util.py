"""Shared helpers of the GPU parity tests (torch = device memory only)."""
from __future__ import annotations

import numpy as np
import torch

from cut_b200 import _lib as L
from cut_b200 import ops


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_l2(got: np.ndarray, ref: np.ndarray) -> float:
    got = got.astype(np.float64)
    ref = ref.astype(np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


def run_blocks(fmt, A_np, W_np, N, *, variant=L.VARIANT_AUTO, D_np=None, fusion_type=0, fusion_op=0, with_status=True, flags=0):
    """C-ABI quantized matmul over GGUF blocks on numpy inputs; returns (C, variant used, status word)."""
    A = dev(A_np)
    W = dev(W_np)
    D = dev(D_np) if D_np is not None else None
    status = torch.zeros(1, dtype=torch.int32, device="cuda") if with_status else None
    d, C_out, keep = ops.make_desc(A, W, fmt, N, D=D, fusion_type=fusion_type, fusion_op=fusion_op, variant=variant,
                                   status=status, flags=flags)
    used = ops.select_variant(d)
    need = ops.workspace_bytes(d)
    ws = None
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        d.workspace, d.workspace_bytes = ws.data_ptr(), need
    ops.launch(d)
    torch.cuda.synchronize()
    st = int(status.item()) if with_status else 0
    return C_out.cpu().numpy(), used, st
