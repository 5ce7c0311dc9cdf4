"""CPU restatement of the reference's definition of the operator.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows z-lab/flash-colreduce ``flash_colreduce/naive.py:8-40`` step by step:

  naive.py:15-17   M, N and the default scale 1/sqrt(D)
  naive.py:19      scores = Q K^T * scale
  naive.py:20-24   right-aligned causal mask: key j is masked for query i when i + max(N-M,0) < j
  naive.py:25      softmax over the key axis
  naive.py:27-37   sum / mean / max over the query axis; the mean divisor is M for the first
                   max(N-M,0) columns (and for every column without the mask) and N-c, ..., 1 after
  naive.py:40      cast to the input dtype

The only liberty taken is blocking: the reference materialises the whole
(B,H,M,N) matrix, this walks it in row blocks (rows are independent -- the
softmax is per row) so that the large benchmark shapes fit in host memory.

Pinning: the reference publishes no golden vectors for this path
(tests/test_correctness.py compares two implementations at run time), so this
oracle is pinned against outputs of the reference's own ``naive_colreduce``
executed in the build container: ``tests/golden/naive_golden.npz``, written by
``tests/golden/make_golden.py``; ``tests/test_oracle.py`` checks it, together
with closed-form cases and the independent C restatement ``colreduce_ref.c``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def oracle_valid_scores(b: int, h: int, m: int, n: int, is_causal: bool) -> int:
    """Number of unmasked (query, key) pairs: B*H*sum_i min(i + max(N-M,0) + 1, N)."""
    if not is_causal:
        return b * h * m * n
    c = max(n - m, 0)
    return b * h * sum(min(i + c + 1, n) for i in range(m))


def oracle_colreduce(
    query: torch.Tensor,
    key: torch.Tensor,
    reduction: str,
    is_causal: bool = False,
    scale: Optional[float] = None,
    compute_dtype: torch.dtype = torch.float32,
    block_rows: int = 2048,
    row_range: Optional[tuple] = None,
    apply_mean: bool = True,
) -> torch.Tensor:
    """Column reduction of softmax(Q K^T * scale) on the CPU in ``compute_dtype``.

    ``row_range=(lo, hi)`` restricts the fold to query rows [lo, hi) of the
    full problem (the mask alignment stays that of the full problem); with
    ``apply_mean=False`` the mean divisor is left out.  Both exist so that a
    bounded sample of a large workload, or one shard of it, can be checked.
    Returns a (B, H, N) tensor of ``compute_dtype``.
    """
    if reduction not in ("sum", "mean", "max"):
        raise ValueError(f"Invalid reduction: {reduction}. Must be 'sum', 'mean', or 'max'.")
    q = query.detach().to("cpu").to(compute_dtype)
    k = key.detach().to("cpu").to(compute_dtype)
    b, h, m, d = q.shape
    n = k.shape[2]
    if scale is None:
        scale = 1 / math.sqrt(d)                                   # naive.py:16-17
    c = max(n - m, 0)                                              # naive.py:21
    lo, hi = (0, m) if row_range is None else row_range
    out = torch.zeros((b, h, n), dtype=compute_dtype)
    k_idx = torch.arange(n).view(1, 1, 1, -1)
    kt = k.transpose(-2, -1)
    for r0 in range(lo, hi, block_rows):
        r1 = min(r0 + block_rows, hi)
        scores = torch.matmul(q[:, :, r0:r1], kt) * scale          # naive.py:19
        if is_causal:
            q_idx = torch.arange(r0, r1).view(1, 1, -1, 1)
            scores = scores.masked_fill(q_idx + c < k_idx, -float("inf"))  # naive.py:22-24
        scores = torch.softmax(scores, dim=-1)                     # naive.py:25
        if reduction == "max":
            out = torch.maximum(out, scores.max(dim=2)[0])         # naive.py:37
        else:
            out += scores.sum(dim=2)                               # naive.py:28,30
    if reduction == "mean" and apply_mean:                         # naive.py:29-35
        if is_causal:
            out[..., :c] /= m
            out[..., c:] /= torch.arange(n - c, 0, -1).to(compute_dtype)
        else:
            out /= m
    return out
