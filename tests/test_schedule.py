"""Tile schedule of the two passes, validated on the CPU.

Work items are decoded by the library (the routine the kernels execute); the
tests check that the items cover exactly the tiles that hold an unmasked score
and that a torch emulation of the tile walk reproduces the oracle.
"""
import itertools

import pytest
import torch

from emulate import TILE, emulate
from oracle import oracle_colreduce

SHAPES = [(128, 128), (131, 131), (128, 1024), (131, 1027), (300, 100), (1, 500), (700, 700), (513, 257), (257, 513),
          (1, 1500), (100, 1027), (128, 4096)]


def _needed_tiles(m, n, causal, off):
    """Set of (query tile, key tile) pairs containing at least one unmasked score."""
    need = set()
    for ti in range((m + TILE - 1) // TILE):
        for tj in range((n + TILE - 1) // TILE):
            if not causal:
                need.add((ti, tj))
                continue
            last_row = min(ti * TILE + TILE, m) - 1
            if tj * TILE <= last_row + off:
                need.add((ti, tj))
    return need


@pytest.mark.parametrize("m,n", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sms", [1, 148, 100000])
def test_items_cover_each_needed_tile_once(m, n, causal, sms):
    q = torch.zeros(1, 2, m, 16).half()
    k = torch.zeros(1, 2, n, 16).half()
    _, pl, visits = emulate(q, k, "sum", causal, num_sms=sms)
    need = _needed_tiles(m, n, causal, pl.causal_offset)
    rows = [(bh, r0 // TILE, t) for (bh, r0, t) in visits[1]]
    cols = [(bh, t, r0 // TILE) for (bh, r0, t) in visits[2]]
    for seen in (rows, cols):
        assert len(seen) == len(set(seen)), "a tile was visited twice"
        for bh in range(2):
            assert {(a, b) for (h, a, b) in seen if h == bh} == need


@pytest.mark.parametrize("m,n", SHAPES)
def test_emulated_walk_matches_oracle(m, n):
    g = torch.Generator().manual_seed(m * 7 + n)
    q = torch.randn(1, 2, m, 24, generator=g).half()
    k = torch.randn(1, 2, n, 24, generator=g).half()
    for red, causal, sms in itertools.product(("sum", "mean", "max"), (False, True), (2, 148)):
        got, _, _ = emulate(q, k, red, causal, num_sms=sms)
        want = oracle_colreduce(q, k, red, causal, compute_dtype=torch.float64)
        torch.testing.assert_close(got.double(), want, rtol=2e-4, atol=1e-6, msg=lambda s: f"{m}x{n} {red} {causal} {sms}: {s}")


def test_negative_scale_and_explicit_offset():
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, 1, 200, 16, generator=g).half()
    k = torch.randn(1, 1, 300, 16, generator=g).half()
    got, _, _ = emulate(q, k, "sum", True, scale=-0.4)
    want = oracle_colreduce(q, k, "sum", True, scale=-0.4, compute_dtype=torch.float64)
    torch.testing.assert_close(got.double(), want, rtol=2e-4, atol=1e-6)
    # a row slice [64, 200) of the problem above, mask offset passed explicitly
    got, _, _ = emulate(q[:, :, 64:], k, "sum", True, scale=0.3, causal_offset=100 + 64)
    want = oracle_colreduce(q, k, "sum", True, scale=0.3, compute_dtype=torch.float64, row_range=(64, 200))
    torch.testing.assert_close(got.double(), want, rtol=2e-4, atol=1e-6)
