"""The operator for inputs that live in host memory.

``flash_colreduce_host`` streams (batch, head) groups through the GPU: while
the kernels reduce one group, the next group's Q and K are copied host to
device on a second stream, and finished (heads, N) results are copied back.
The arithmetic is that of :func:`flash_colreduce_b200.flash_colreduce`, group
by group (heads are independent, flash_colreduce/flash.py:169-175).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .op import flash_colreduce

__all__ = ["flash_colreduce_host", "release_host_buffers"]


def flash_colreduce_host(
    query: torch.Tensor,
    key: torch.Tensor,
    reduction: str,
    is_causal: bool = False,
    scale: Optional[float] = None,
    *,
    device: Optional[torch.device] = None,
    group_heads: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Column reduction of host-resident (ideally pinned) ``query`` / ``key``.

    Returns a host tensor (B, H, N) of ``query.dtype`` (``out`` if given).  The
    call returns after the last result has reached the host.
    """
    if query.is_cuda or key.is_cuda:
        raise ValueError("flash_colreduce_host takes host tensors; use flash_colreduce for CUDA tensors")
    if not all(query.shape[i] == key.shape[i] for i in [0, 1, 3]):
        raise ValueError(
            f"Query and key tensors must have same batch size, number of heads, and head dimension. "
            f"Got query shape: {query.shape}, key shape: {key.shape}."
        )
    if reduction not in ["sum", "mean", "max"]:
        raise ValueError(f"Invalid reduction: {reduction}. Must be 'sum', 'mean', or 'max'.")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    b, h, m, d = query.shape
    n = key.shape[2]
    if scale is None:
        scale = 1 / math.sqrt(d)
    if out is None:
        out = torch.empty((b, h, n), dtype=query.dtype, pin_memory=True)
    if out.numel() == 0:
        return out
    ramp = group_heads is None
    if ramp:
        # About eight groups per batch entry, capped at 512 MiB of input, so that every launch
        # carries many heads.  The first group's copy is the only one that is not hidden behind
        # kernels: the very first groups are small (1, 1, 2, 4, ... heads) and grow to that size.
        per_head = (m + n) * d * query.element_size()
        group_heads = max(1, min(-(-h // 8), (512 << 20) // max(per_head, 1)))
    groups = []
    for bi in range(b):
        h0, size = 0, (1 if ramp and bi == 0 else group_heads)
        while h0 < h:
            groups.append((bi, h0, min(h0 + size, h)))
            h0 += size
            if len(groups) >= 2:
                size = min(2 * size, group_heads)
    with torch.cuda.device(device):
        compute = torch.cuda.current_stream(device)
        ctx = _context(device, min(group_heads, h), m, n, d, query.dtype)
        copier, bufs, loaded, consumed = ctx.copier, ctx.bufs, ctx.loaded, ctx.consumed
        # The staging buffers may still be read by kernels of an earlier call on the compute
        # stream (or, freshly allocated, by whatever last used their memory): the copy stream
        # starts behind everything queued on the compute stream so far.
        copier.wait_stream(compute)

        def load(idx):
            bi, h0, h1 = groups[idx]
            slot = idx % 2
            with torch.cuda.stream(copier):
                if idx >= 2:
                    copier.wait_event(consumed[slot])
                bufs[slot][0][:, : h1 - h0].copy_(query[bi : bi + 1, h0:h1], non_blocking=True)
                bufs[slot][1][:, : h1 - h0].copy_(key[bi : bi + 1, h0:h1], non_blocking=True)
                loaded[slot].record(copier)

        load(0)
        for idx, (bi, h0, h1) in enumerate(groups):
            slot = idx % 2
            if idx + 1 < len(groups):
                load(idx + 1)
            compute.wait_event(loaded[slot])
            res = flash_colreduce(bufs[slot][0][:, : h1 - h0], bufs[slot][1][:, : h1 - h0], reduction,
                                  is_causal=is_causal, scale=scale)
            consumed[slot].record(compute)
            out[bi, h0:h1].copy_(res[0], non_blocking=True)
        compute.synchronize()
    return out


class _HostContext:
    """Copy stream, two pairs of device staging buffers and their events, kept between calls."""

    def __init__(self, device, gh, m, n, d, dtype):
        self.copier = torch.cuda.Stream(device)
        self.bufs = [(torch.empty((1, gh, m, d), dtype=dtype, device=device),
                      torch.empty((1, gh, n, d), dtype=dtype, device=device)) for _ in range(2)]
        self.loaded = [torch.cuda.Event() for _ in range(2)]
        self.consumed = [torch.cuda.Event() for _ in range(2)]


_CONTEXTS: dict = {}


def _context(device, gh, m, n, d, dtype) -> _HostContext:
    """The staging context for a call signature.  One is kept per device (the last signature
    used): repeated calls of one shape, the streaming use this function is for, create no
    stream, buffer or event after the first."""
    sig = (gh, m, n, d, dtype)
    hit = _CONTEXTS.get(device)
    if hit is None or hit[0] != sig:
        _CONTEXTS.pop(device, None)  # release the old buffers before the new ones are allocated
        hit = _CONTEXTS[device] = (sig, _HostContext(device, gh, m, n, d, dtype))
    return hit[1]


def release_host_buffers() -> None:
    """Frees the device staging buffers ``flash_colreduce_host`` keeps between calls."""
    _CONTEXTS.clear()
