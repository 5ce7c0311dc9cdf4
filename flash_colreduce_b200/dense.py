"""``naive_colreduce`` -- the materialising definition of the operator.

Part of the public API because the reference exports it
(flash_colreduce/naive.py:8-40); it is the plain-PyTorch statement of what
``flash_colreduce`` computes and runs on whatever device its inputs are on.
Rows are processed in blocks so that a block of the (M, N) matrix, not all of
it, is alive at a time; the arithmetic per row is the definition's.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

__all__ = ["naive_colreduce"]


def naive_colreduce(
    query: torch.Tensor,
    key: torch.Tensor,
    reduction: str,
    is_causal: bool = False,
    scale: Optional[float] = None,
    block_rows: int = 4096,
) -> torch.Tensor:
    if reduction not in ("sum", "mean", "max"):
        raise ValueError(f"Invalid reduction: {reduction}. Must be 'sum', 'mean', or 'max'.")
    m, n = query.shape[2], key.shape[2]
    if scale is None:
        scale = 1 / math.sqrt(query.shape[-1])
    shift = max(n - m, 0)
    key_t = key.transpose(-2, -1)
    key_pos = torch.arange(n, device=query.device)
    folded = torch.zeros(query.shape[:2] + (n,), dtype=query.dtype, device=query.device)
    for lo in range(0, m, max(int(block_rows), 1)):
        hi = min(lo + block_rows, m)
        att = torch.matmul(query[:, :, lo:hi], key_t) * scale
        if is_causal:
            row_pos = torch.arange(lo, hi, device=query.device)
            att = att.masked_fill(row_pos[:, None] + shift < key_pos[None, :], -float("inf"))
        att = torch.softmax(att, dim=-1)
        if reduction == "max":
            folded = torch.maximum(folded, att.max(dim=2)[0])
        else:
            folded = folded + att.sum(dim=2)
    if reduction == "mean":
        if is_causal:
            folded[..., :shift] /= m
            folded[..., shift:] /= torch.arange(n - shift, 0, -1, device=query.device)
        else:
            folded /= m
    return folded.to(query.dtype)
