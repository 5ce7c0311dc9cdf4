"""CPU emulation of the two-pass tile walk of the sm_100a kernels.

The work items come from the library's own ``fcr_plan_item`` (the routine the
kernels run); the per-tile arithmetic and the mask predicates are restated here
in torch, tile by tile, so that the schedule (tile ranges, splits, masks,
partial combination) can be validated on a machine without a GPU.
"""
from __future__ import annotations

import math

import torch

from flash_colreduce_b200 import _native as nat

TILE = 128


def emulate(q: torch.Tensor, k: torch.Tensor, reduction: str, is_causal: bool, scale=None, num_sms: int = 148,
            causal_offset: int = -1):
    """Returns (fp32 result (B,H,N), plan, tile-visit log)."""
    B, H, M, D = q.shape
    N = k.shape[2]
    if scale is None:
        scale = 1 / math.sqrt(D)
    prob = nat.make_problem(B, H, M, N, D, q.stride(), k.stride(), nat.FCR_F16, nat.REDUCTION_CODES[reduction],
                            is_causal, scale, causal_offset)
    pl = nat.plan(prob, num_sms)
    off = pl.causal_offset
    scale2 = abs(scale) * 1.4426950408889634
    sign = -1.0 if scale < 0 else 1.0
    qf = q.float().reshape(B * H, M, D)
    kf = k.float().reshape(B * H, N, D)
    qpad = torch.zeros(B * H, pl.m_pad + TILE, D)
    kpad = torch.zeros(B * H, pl.n_pad + TILE, D)
    qpad[:, :M] = qf
    kpad[:, :N] = kf
    visits = {1: [], 2: []}

    # rows pass
    part_m = torch.full((pl.row_splits, B * H, pl.m_pad), float("-inf"))
    part_l = torch.zeros((pl.row_splits, B * H, pl.m_pad))
    for item in range(pl.row_items):
        it = nat.plan_item(prob, pl, 1, item)
        bh = it["head"]
        if pl.key_stream:
            # key streaming: warpgroup w folds tiles t_lo + w, t_lo + w + 4, ... into partial slot 4 * chunk + w
            lo, hi = it["chunk"]
            assert it["sub"][0] == (0, lo, hi) and it["sub"][1][1] == it["sub"][1][2]
            walks = [(4 * it["split"] + w, 0, list(range(lo + w, hi, 4))) for w in range(4)]
        else:
            walks = [(it["split"], r0, list(range(t_lo, t_hi))) for (r0, t_lo, t_hi) in it["sub"]]
            for (r0, t_lo, t_hi) in it["sub"]:
                assert t_lo == t_hi if r0 >= M else True
        for (sp, r0, tiles) in walks:
            if r0 >= M:
                continue
            rows = torch.arange(r0, r0 + TILE)
            m_run = torch.full((TILE,), float("-inf"))
            l_run = torch.zeros(TILE)
            for t in tiles:
                assert it["chunk"][0] <= t < it["chunk"][1]
                visits[1].append((bh, r0, t))
                c0 = t * TILE
                s = sign * (qpad[bh, r0:r0 + TILE] @ kpad[bh, c0:c0 + TILE].T)
                need_mask = (c0 + TILE > N) or (is_causal and (c0 + TILE - 1 > r0 + off))
                x = s * scale2
                if need_mask:
                    jlim = torch.clamp(rows + off, max=N - 1) if is_causal else torch.full((TILE,), N - 1)
                    cols = torch.arange(c0, c0 + TILE)
                    x = torch.where(cols[None, :] <= jlim[:, None], x, torch.tensor(float("-inf")))
                m_new = torch.maximum(m_run, x.max(dim=1)[0])
                m_safe = torch.where(torch.isinf(m_new), torch.zeros(()), m_new)
                l_run = l_run * torch.exp2(m_run - m_safe) + torch.exp2(x - m_safe[:, None]).sum(dim=1)
                m_run = m_new
            part_m[sp, bh, r0:r0 + TILE] = m_run
            part_l[sp, bh, r0:r0 + TILE] = l_run
    mx = part_m.max(dim=0)[0]
    w = torch.where(torch.isinf(part_m), torch.zeros(()), torch.exp2(part_m - mx[None]))
    neg_lse = -(mx + torch.log2((part_l * w).sum(dim=0)))

    # columns pass
    is_max = reduction == "max"
    part_out = torch.zeros((pl.col_splits, B * H, pl.n_pad))
    for item in range(pl.col_items):
        it = nat.plan_item(prob, pl, 2, item)
        bh, sp = it["head"], it["split"]
        if pl.key_stream:
            # key streaming: every key tile of the chunk against the head's single query tile
            sp = 0
            subs = [(kt * TILE, 0, 1) for kt in range(*it["chunk"])]
        else:
            subs = it["sub"]
        for (r0, t_lo, t_hi) in subs:
            if r0 >= N:
                assert t_lo == t_hi
                continue
            keys = torch.arange(r0, r0 + TILE)
            acc = torch.full((TILE,), float("-inf")) if is_max else torch.zeros(TILE)
            for t in range(t_lo, t_hi):
                assert pl.key_stream or it["chunk"][0] <= t < it["chunk"][1]
                visits[2].append((bh, r0, t))
                c0 = t * TILE
                s = sign * (kpad[bh, r0:r0 + TILE] @ qpad[bh, c0:c0 + TILE].T)  # (keys, queries)
                nl = torch.zeros(TILE)
                hi = min(c0 + TILE, pl.m_pad)
                nl[: hi - c0] = neg_lse[bh, c0:hi]
                x = s * scale2 + nl[None, :]
                need_mask = (c0 + TILE > M) or (is_causal and (c0 + off < r0 + TILE - 1))
                if need_mask:
                    qi = torch.arange(c0, c0 + TILE)
                    lo = torch.clamp(keys - off, min=0) if is_causal else torch.zeros(TILE, dtype=torch.long)
                    valid = (qi[None, :] >= lo[:, None]) & (qi[None, :] < M)
                else:
                    valid = torch.ones(TILE, TILE, dtype=torch.bool)
                if is_max:
                    acc = torch.maximum(acc, torch.where(valid, x, torch.tensor(float("-inf"))).max(dim=1)[0])
                else:
                    acc = acc + torch.where(valid, torch.exp2(x), torch.zeros(())).sum(dim=1)
            part_out[sp, bh, r0:r0 + TILE] = torch.exp2(acc) if is_max else acc
    res = part_out.max(dim=0)[0] if is_max else part_out.sum(dim=0)
    res = res[:, :N]
    if reduction == "mean":
        if is_causal:
            c = max(N - M, 0)
            div = torch.full((N,), float(M))
            div[c:] = torch.arange(N - c, 0, -1).float()
        else:
            div = torch.full((N,), float(M))
        res = res / div
    return res.reshape(B, H, N), pl, visits
