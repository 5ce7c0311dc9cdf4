"""``flash_colreduce`` -- the public operator, backed by the sm_100a library.

Same signature, semantics, output shape/dtype and error messages as the
reference operator (flash_colreduce/flash.py:311-385).  All device work is
done by hand-written CUDA kernels reached through the C ABI; there is no
Triton path and no CPU or eager fallback.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch

from . import _native as nat

__all__ = ["flash_colreduce", "colreduce_partial", "finalize_scores", "valid_scores", "topk_columns",
           "flash_colreduce_topk", "select_columns"]

_DTYPE_CODES = {torch.float16: nat.FCR_F16, torch.bfloat16: nat.FCR_BF16, torch.float32: nat.FCR_F32}


def _debug_sync() -> bool:
    return os.environ.get("FCR_DEBUG_SYNC", "0") not in ("", "0")


def _tma_ready(x: torch.Tensor) -> torch.Tensor:
    """Returns ``x`` or a copy whose layout a TMA tensor map can describe.

    Needed: innermost stride 1, every other stride of a dimension longer than
    one a positive multiple of 16 bytes, 16-byte aligned base.  The head
    dimension is zero-padded to a multiple of 16 bytes when it is not one,
    which changes no dot product (the reference pads to a power of two for the
    same reason, flash_colreduce/flash.py:368-373).
    """
    d = x.shape[-1]
    unit = 16 // x.element_size()  # elements per 16 bytes: 8 for fp16 / bf16, 4 for fp32
    if d % unit != 0:
        x = torch.nn.functional.pad(x, (0, unit - d % unit))
    ok = x.stride(3) == 1 and x.data_ptr() % 16 == 0
    for dim in range(3):
        if x.shape[dim] > 1 and (x.stride(dim) <= 0 or x.stride(dim) % unit != 0):
            ok = False
    return x if ok else x.contiguous()


_PLAN_CACHE: dict = {}


def _problem_and_workspace_bytes(key_tuple, device):
    """Problem struct and workspace size for a call signature (cached: planning is pure host work)."""
    hit = _PLAN_CACHE.get(key_tuple)
    if hit is None:
        (b, h, m, n, d, qs, ks, dt, red, causal, scale, off, mean_m, mean_n, _dev) = key_tuple
        prob = nat.make_problem(b, h, m, n, d, qs, ks, dt, red, causal, scale, off, mean_m, mean_n)
        with torch.cuda.device(device):
            pl = nat.plan(prob, 0)
        if len(_PLAN_CACHE) > 4096:
            _PLAN_CACHE.clear()
        hit = _PLAN_CACHE[key_tuple] = (prob, int(pl.workspace_bytes))
    return hit


def _launch(query, key, out, out_code, reduction_code, is_causal, scale, causal_offset, mean_M, mean_N):
    """Plans (cached), allocates the workspace and queues the kernels on the current stream.

    No synchronisation.  A bounded wait that expired inside a kernel of an EARLIER call on this
    device is reported here: the library finds the status in its mailbox in mapped host memory
    and returns FCR_ERR_DEVICE_TIMEOUT instead of launching, which ``nat.check`` turns into a
    ``RuntimeError``.  ``FCR_DEBUG_SYNC=1`` additionally synchronises after every call and reads
    the status words of the call's own workspace.
    """
    b, h, m, _ = query.shape
    n = key.shape[2]
    q = _tma_ready(query)
    k = _tma_ready(key)
    d = q.shape[-1]
    prob, ws_bytes = _problem_and_workspace_bytes(
        (b, h, m, n, d, tuple(q.stride()), tuple(k.stride()), _DTYPE_CODES[q.dtype], reduction_code, bool(is_causal),
         float(scale), int(causal_offset), int(mean_M), int(mean_N), q.device.index), q.device)
    with torch.cuda.device(q.device):
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        stream = torch.cuda.current_stream(q.device).cuda_stream
        rc = nat.lib.fcr_colreduce(C.byref(prob), q.data_ptr(), k.data_ptr(), out.data_ptr(), out_code,
                                   ws.data_ptr(), ws.numel(), stream)
        nat.check(rc, "fcr_colreduce")
        if _debug_sync():
            nat.check(nat.lib.fcr_read_device_status(ws.data_ptr(), stream, None), "fcr_colreduce (device)")
    return out


def _validate(query: torch.Tensor, key: torch.Tensor, reduction: str) -> None:
    if not query.is_cuda or not key.is_cuda:
        raise ValueError("Query and key tensors must be on CUDA device.")
    if not all(query.shape[i] == key.shape[i] for i in [0, 1, 3]):
        raise ValueError(
            f"Query and key tensors must have same batch size, number of heads, and head dimension. "
            f"Got query shape: {query.shape}, key shape: {key.shape}."
        )
    if reduction not in ["sum", "mean", "max"]:
        raise ValueError(f"Invalid reduction: {reduction}. Must be 'sum', 'mean', or 'max'.")
    if query.dtype != key.dtype or query.dtype not in _DTYPE_CODES:
        raise TypeError(
            f"flash_colreduce takes fp16, bf16 or fp32 (run as TF32) tensors of one dtype; "
            f"got query {query.dtype}, key {key.dtype}."
        )
    d_max = 512 // query.element_size()
    if query.shape[-1] > d_max:
        raise ValueError(f"Head dimension {query.shape[-1]} exceeds {d_max}, the largest the sm_100a kernels take "
                         f"for {query.dtype} (operand rows of at most 512 bytes).")


def flash_colreduce(
    query: torch.Tensor,
    key: torch.Tensor,
    reduction: str,
    is_causal: bool = False,
    scale: Optional[float] = None,
) -> torch.Tensor:
    """Column reduction of the softmax attention matrix, never materialised.

    ``S = softmax(Q K^T * scale)`` per (batch, head) and query row;
    ``R[b, h, n] = reduce_m S[b, h, m, n]`` with ``reduce`` one of ``"sum"``,
    ``"mean"``, ``"max"``.  With ``is_causal`` the mask is right-aligned:
    query ``m`` attends keys up to ``m + max(N - M, 0)``; ``"mean"`` divides a
    column by the number of queries the reference counts for it
    (flash_colreduce/flash.py:377-384: ``M`` for the first ``max(N - M, 0)``
    columns, then ``N - n``).

    Args:
        query: (B, H, M, D) CUDA tensor: fp16 or bf16 with D <= 256, or fp32 with D <= 128
            (fp32 operands are multiplied as TF32, like the reference's tl.dot).  Rows of up to
            256 bytes (D <= 128 in 16 bits) run the fast path.
        key: (B, H, N, D), same dtype and device.
        reduction: "sum", "mean" or "max".
        is_causal: apply the right-aligned causal mask.
        scale: softmax scale, default ``1 / sqrt(D)``.

    Returns:
        (B, H, N) tensor of ``query.dtype``.  Accumulation is fp32 and the
        result is rounded once; run-to-run results are bitwise identical.
    """
    _validate(query, key, reduction)
    b, h, m, d = query.shape
    n = key.shape[2]
    if scale is None:
        scale = 1 / math.sqrt(d)
    out = torch.empty((b, h, n), dtype=query.dtype, device=query.device)
    if out.numel() == 0:
        return out
    if m == 0:
        # no query contributes: zeros for sum / max, 0/0 for mean as in the reference
        out.zero_()
        return out / 0 if reduction == "mean" else out
    return _launch(query, key, out, _DTYPE_CODES[out.dtype], nat.REDUCTION_CODES[reduction], is_causal,
                   scale, -1, 0, 0)


def colreduce_partial(
    query: torch.Tensor,
    key: torch.Tensor,
    reduction: str,
    is_causal: bool,
    scale: float,
    causal_offset: int,
) -> torch.Tensor:
    """fp32 column sums (``"sum"``) or maxima (``"max"``) of a row slice.

    ``query`` holds a slice of the rows of a larger problem; row ``i`` of the
    slice attends keys ``j <= i + causal_offset``.  No mean divisor, no cast:
    shards are combined with ``+`` / ``max`` and passed to
    :func:`finalize_scores`.  Used by the multi-GPU driver.
    """
    _validate(query, key, reduction)
    if reduction == "mean":
        raise ValueError("colreduce_partial takes 'sum' or 'max'; apply the mean in finalize_scores")
    b, h, m, _ = query.shape
    n = key.shape[2]
    out = torch.empty((b, h, n), dtype=torch.float32, device=query.device)
    if out.numel() == 0 or m == 0:
        return out.zero_()
    return _launch(query, key, out, nat.FCR_F32, nat.REDUCTION_CODES[reduction], is_causal, scale,
                   causal_offset if is_causal else -1, 0, 0)


def finalize_scores(acc: torch.Tensor, m: int, reduction: str, is_causal: bool, dtype: torch.dtype) -> torch.Tensor:
    """Mean divisor (flash_colreduce/flash.py:377-384) and cast of fp32 (B,H,N) sums / maxima."""
    if acc.dtype != torch.float32 or not acc.is_cuda or not acc.is_contiguous():
        raise ValueError("acc must be a contiguous fp32 CUDA tensor")
    b, h, n = acc.shape
    out = torch.empty((b, h, n), dtype=dtype, device=acc.device)
    if out.numel() == 0:
        return out
    with torch.cuda.device(acc.device):
        stream = torch.cuda.current_stream(acc.device).cuda_stream
        rc = nat.lib.fcr_finalize(acc.data_ptr(), out.data_ptr(), _DTYPE_CODES[dtype], b, h, m, n,
                                  nat.REDUCTION_CODES[reduction], 1 if is_causal else 0, stream)
        nat.check(rc, "fcr_finalize")
    return out


def topk_columns(scores: torch.Tensor, k: int, return_values: bool = True):
    """The ``k`` highest-scoring key positions of every (batch, head) row of ``scores`` (..., N).

    Returns ``(values, indices)`` like ``torch.topk`` (``values`` is ``None`` when not asked for), but
    in ascending position order -- the order a token-pruning consumer gathers in -- and with ties at
    the k-th score resolved towards the lowest positions.  One kernel launch on the current stream.
    The reference stops at the scores (its README.md:9 names this use); there is no counterpart.
    """
    if not scores.is_cuda:
        raise ValueError("scores must be on a CUDA device.")
    if scores.dtype not in _DTYPE_CODES:
        raise TypeError(f"topk_columns takes fp16, bf16 or fp32 scores; got {scores.dtype}.")
    n = scores.shape[-1]
    if not 1 <= k <= n:
        raise ValueError(f"k = {k} must lie in [1, {n}].")
    flat = scores.contiguous().view(-1, n)
    lead = scores.shape[:-1]
    indices = torch.empty((flat.shape[0], k), dtype=torch.int64, device=scores.device)
    values = torch.empty((flat.shape[0], k), dtype=scores.dtype, device=scores.device) if return_values else None
    if flat.shape[0] > 0:
        with torch.cuda.device(scores.device):
            stream = torch.cuda.current_stream(scores.device).cuda_stream
            rc = nat.lib.fcr_topk(flat.data_ptr(), _DTYPE_CODES[scores.dtype], flat.shape[0], n, k,
                                  indices.data_ptr(), 64, values.data_ptr() if return_values else None, stream)
            nat.check(rc, "fcr_topk")
    return (values.view(*lead, k) if return_values else None), indices.view(*lead, k)


def select_columns(scores: torch.Tensor, threshold: float):
    """Key positions whose score exceeds ``threshold``, per (batch, head) row of ``scores`` (..., N).

    Returns ``(indices, counts)``: ``indices`` (..., N) int64 holds, for every row, the selected
    positions in ascending order in its first ``counts[...]`` entries (the rest is unspecified), ``counts``
    (...) int32.  One kernel launch on the current stream; the reference has no counterpart.
    """
    if not scores.is_cuda:
        raise ValueError("scores must be on a CUDA device.")
    if scores.dtype not in _DTYPE_CODES:
        raise TypeError(f"select_columns takes fp16, bf16 or fp32 scores; got {scores.dtype}.")
    n = scores.shape[-1]
    flat = scores.contiguous().view(-1, n)
    lead = scores.shape[:-1]
    indices = torch.empty((flat.shape[0], n), dtype=torch.int64, device=scores.device)
    counts = torch.zeros((flat.shape[0],), dtype=torch.int32, device=scores.device)
    if flat.numel() > 0:
        with torch.cuda.device(scores.device):
            stream = torch.cuda.current_stream(scores.device).cuda_stream
            rc = nat.lib.fcr_select_above(flat.data_ptr(), _DTYPE_CODES[scores.dtype], flat.shape[0], n, float(threshold),
                                          indices.data_ptr(), 64, counts.data_ptr(), stream)
            nat.check(rc, "fcr_select_above")
    return indices.view(*lead, n), counts.view(*lead)


def flash_colreduce_topk(query: torch.Tensor, key: torch.Tensor, reduction: str, k: int, is_causal: bool = False,
                         scale: Optional[float] = None):
    """``flash_colreduce`` followed by :func:`topk_columns`: ``(values, indices)`` of shape (B, H, k)."""
    return topk_columns(flash_colreduce(query, key, reduction, is_causal=is_causal, scale=scale), k)


def valid_scores(b: int, h: int, m: int, n: int, is_causal: bool) -> int:
    """Number of unmasked attention scores of a problem: the unit of the throughput metric."""
    if not is_causal:
        return b * h * m * n
    off = max(n - m, 0)
    ramp = max(0, min(m, n - off))
    return b * h * (ramp * (off + 1) + ramp * (ramp - 1) // 2 + (m - ramp) * n)
