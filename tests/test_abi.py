"""The C-ABI library: exported symbols, host-side planner and error reporting (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

from flash_colreduce_b200 import _native as nat

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _contig(b, h, rows, d):
    return (h * rows * d, rows * d, d, 1)


def _problem(b, h, m, n, d, red="sum", causal=False, scale=0.125, **kw):
    return nat.make_problem(b, h, m, n, d, _contig(b, h, m, d), _contig(b, h, n, d), nat.FCR_F16,
                            nat.REDUCTION_CODES[red], causal, scale, **kw)


def test_every_declared_symbol_is_exported():
    header = open(os.path.join(ROOT, "include", "flash_colreduce_b200.h")).read()
    declared = set(re.findall(r"\b(fcr_[a-z0-9_]+)\s*\(", header))
    assert declared == set(nat.EXPORTS)
    for name in declared:
        assert getattr(nat.lib, name) is not None


def test_version():
    assert nat.lib.fcr_version().decode() == "0.1.0"


# (B, H, M, N, D, causal) -> scores of the benchmark configurations
CONFIG_SCORES = [
    ((2, 4, 256, 256, 64, False), 524_288),
    ((8, 16, 512, 512, 64, False), 33_554_432),
    ((1, 32, 128, 4096, 128, True), 16_517_120),
    ((4, 32, 8192, 8192, 128, True), 4_295_491_584),
    ((1, 64, 131072, 131072, 128, True), 549_760_008_192),
]


@pytest.mark.parametrize("cfg,scores", CONFIG_SCORES)
def test_plan_counts_valid_scores(cfg, scores):
    b, h, m, n, d, causal = cfg
    pl = nat.plan(_problem(b, h, m, n, d, causal=causal), 148)
    assert pl.valid_scores == scores
    assert pl.d_pad == (64 if d <= 64 else 128 if d <= 128 else 256)
    assert pl.m_pad % 128 == 0 and pl.m_pad >= m and pl.n_pad % 128 == 0 and pl.n_pad >= n
    if pl.key_stream:  # decode shape: key chunks are the work items of both passes
        assert (m, n) == (128, 4096) and pl.key_chunks >= 1
        assert pl.row_items == pl.col_items == b * h * pl.key_chunks
        assert pl.row_splits == 4 * pl.key_chunks and pl.col_splits == 1
    else:
        assert pl.row_items == b * h * pl.row_blocks * pl.row_splits
        assert pl.col_items == b * h * pl.col_blocks * pl.col_splits
    assert 1 <= pl.row_ctas <= 148 and 1 <= pl.col_ctas <= 148
    assert pl.workspace_bytes >= 256 + b * h * pl.m_pad * 4
    assert nat.lib.fcr_workspace_bytes(C.byref(_problem(b, h, m, n, d, causal=causal)), 148) == pl.workspace_bytes


def test_small_problems_are_split_to_fill_the_gpu():
    # decode shape: one row block per head, 32 key tiles -> the key range is split
    pl = nat.plan(_problem(1, 32, 128, 4096, 128, causal=True), 148)
    assert pl.row_blocks == 1 and pl.row_splits > 1
    assert pl.off_part_m > 0 and pl.off_part_l > pl.off_part_m
    # plenty of blocks: no split, no partial buffers, items drawn from a counter
    pl = nat.plan(_problem(4, 32, 8192, 8192, 128, causal=True), 148)
    assert pl.row_splits == 1 and pl.col_splits == 1 and pl.off_part_out == 0 and pl.static_schedule == 0
    # at most two items per CTA: dealt round-robin, nothing to clear
    assert nat.plan(_problem(8, 16, 512, 512, 64), 148).static_schedule == 1


def test_decode_plans_stream_the_keys():
    # one query tile, 256 key tiles: key streaming; the last fields of the struct line up with the C layout
    pl = nat.plan(_problem(8, 32, 64, 32768, 128, causal=True), 148)
    assert pl.key_stream == 1 and pl.key_chunks >= 1 and pl.score_cache == 0 and pl.off_scores == 0 and pl.static_schedule == 1
    assert pl.row_splits == 4 * pl.key_chunks and pl.col_splits == 1
    assert pl.row_items == pl.col_items == 8 * 32 * pl.key_chunks
    # at most 16 queries: the raw scores are cached at the end of the workspace
    pl = nat.plan(_problem(8, 32, 4, 32768, 128, causal=True), 148)
    assert pl.key_stream == 1 and pl.score_cache == 1
    assert pl.workspace_bytes - pl.off_scores == 8 * 32 * 4 * pl.n_pad * 4
    # too few key tiles, or more than one query tile: the general kernels
    assert nat.plan(_problem(8, 32, 64, 512, 128, causal=True), 148).key_stream == 0
    assert nat.plan(_problem(8, 32, 129, 32768, 128, causal=True), 148).key_stream == 0
    # every key tile belongs to exactly one work item of its head
    pr = _problem(1, 3, 16, 5000, 64, causal=False)
    pl = nat.plan(pr, 148)
    for which in (1, 2):
        seen = {}
        for item in range(pl.row_items):
            it = nat.plan_item(pr, pl, which, item)
            for t in range(*it["chunk"]):
                assert (it["head"], t) not in seen
                seen[(it["head"], t)] = item
        assert len(seen) == 3 * (pl.n_pad // 128)


def test_causal_offset_defaults_to_right_alignment():
    assert nat.plan(_problem(1, 1, 128, 1024, 64, causal=True), 148).causal_offset == 896
    assert nat.plan(_problem(1, 1, 1024, 128, 64, causal=True), 148).causal_offset == 0
    assert nat.plan(_problem(1, 1, 128, 1024, 64, causal=True, causal_offset=5), 148).causal_offset == 5
    assert nat.plan(_problem(1, 1, 128, 1024, 64, causal=False), 148).causal_offset == 0


@pytest.mark.parametrize(
    "kwargs,status,text",
    [
        (dict(m=0), nat.FCR_ERR_BAD_ARG, "positive"),
        (dict(d=264), nat.FCR_ERR_UNSUPPORTED, "exceeds 256"),
        (dict(dtype=nat.FCR_F32, d=132), nat.FCR_ERR_UNSUPPORTED, "exceeds 128"),
        (dict(dtype=5), nat.FCR_ERR_UNSUPPORTED, "fp16, bf16 or fp32"),
        (dict(red=7), nat.FCR_ERR_BAD_ARG, "invalid reduction"),
        (dict(qs=(0, 0, 72, 2)), nat.FCR_ERR_UNSUPPORTED, "innermost stride"),
        (dict(qs=(0, 0, 20, 1)), nat.FCR_ERR_UNSUPPORTED, "multiple of 8"),
    ],
)
def test_plan_rejects_bad_problems(kwargs, status, text):
    m = kwargs.get("m", 64)
    d = kwargs.get("d", 64)
    p = nat.make_problem(1, 1, m, 64, d, kwargs.get("qs", _contig(1, 1, m, d)), _contig(1, 1, 64, d),
                         kwargs.get("dtype", nat.FCR_F16), kwargs.get("red", 0), False, 0.125)
    pl = nat.Plan()
    rc = nat.lib.fcr_plan_problem(C.byref(p), 148, C.byref(pl))
    assert rc == status
    assert text in nat.last_error()
    assert nat.lib.fcr_workspace_bytes(C.byref(p), 148) == 0


def test_null_arguments_are_rejected_before_any_device_work():
    p = _problem(1, 1, 64, 64, 64)
    assert nat.lib.fcr_colreduce(C.byref(p), None, None, None, nat.FCR_F16, None, 0, None) == nat.FCR_ERR_BAD_ARG
    assert nat.lib.fcr_plan_problem(None, 148, None) == nat.FCR_ERR_BAD_ARG
    assert nat.lib.fcr_finalize(None, None, 0, 1, 1, 1, 1, 0, 0, None) == nat.FCR_ERR_BAD_ARG
    assert nat.lib.fcr_read_device_status(None, None, None) == nat.FCR_ERR_BAD_ARG
    assert nat.lib.fcr_self_test_hooks(-1, 0) == nat.FCR_ERR_BAD_ARG
    assert nat.lib.fcr_self_test_hooks(0, -1) == nat.FCR_OK
    with pytest.raises(RuntimeError, match="status 1"):
        nat.check(nat.FCR_ERR_BAD_ARG, "demo")


def test_launch_counter_starts_at_zero_without_a_gpu():
    import torch

    if not torch.cuda.is_available():
        assert nat.lib.fcr_launch_count() == 0


def test_the_probe_library_exports_its_one_symbol():
    from flash_colreduce_b200.build import PROBE_PATH

    assert C.CDLL(PROBE_PATH).fcr_probe_ex2_rate is not None


def test_plan_item_bounds():
    p = _problem(1, 2, 300, 300, 64, causal=True)
    pl = nat.plan(p, 4)
    buf = (C.c_int32 * 10)()
    assert nat.lib.fcr_plan_item(C.byref(p), C.byref(pl), 1, pl.row_items, buf) == nat.FCR_ERR_BAD_ARG
    assert nat.lib.fcr_plan_item(C.byref(p), C.byref(pl), 3, 0, buf) == nat.FCR_ERR_BAD_ARG
    assert nat.lib.fcr_plan_item(C.byref(p), C.byref(pl), 2, 0, buf) == nat.FCR_OK
