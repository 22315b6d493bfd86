"""MoE routing primitives on raw tensors: top-k, expert plan, gather / combine, grouped GEMM."""
from __future__ import annotations

import torch


def topk(x: torch.Tensor, k: int):
    """Descending top-k of each row, ties to the lower index. Returns (values, int32 indices)."""
    xf = x.float()
    # stable sort on (-value, index) gives the lower index first among equal values
    idx = torch.sort(-xf, dim=1, stable=True).indices[:, :k]
    vals = torch.gather(x, 1, idx)
    return vals, idx.to(torch.int32)
