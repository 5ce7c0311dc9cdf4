"""Parity of the sm_100a kernels with the oracle and the reference's outputs (needs a B200)."""
import math
import os

import pytest
import torch

from conftest import assert_parity
from oracle import oracle_colreduce

pytestmark = pytest.mark.gpu

os.environ.setdefault("FCR_DEBUG_SYNC", "1")  # read the device status words after every call


def _dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def _f32(q, k, red, causal, scale=None):
    """The operator with an fp32 result (mean included): the kernels' accumulators, unrounded."""
    from flash_colreduce_b200 import _native as nat
    from flash_colreduce_b200 import op

    if scale is None:
        scale = 1 / math.sqrt(q.shape[-1])
    out = torch.empty(q.shape[0], q.shape[1], k.shape[2], dtype=torch.float32, device=q.device)
    return op._launch(q, k, out, nat.FCR_F32, nat.REDUCTION_CODES[red], causal, scale, -1, 0, 0)


def _rand(shape, seed, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)


def test_native_library_is_loaded():
    from flash_colreduce_b200 import _native as nat

    from flash_colreduce_b200.ex2_probe import ex2_rate

    assert nat.lib.fcr_version().decode() == "0.1.0"
    before = nat.lib.fcr_launch_count()
    _f32(_rand((1, 1, 64, 64), 1).to(_dev()), _rand((1, 1, 64, 64), 2).to(_dev()), "sum", False)
    assert nat.lib.fcr_launch_count() - before >= 2  # the two pass kernels at least
    assert ex2_rate(1) > 1e12


def test_golden_vectors_fp32(golden):
    """Every output of the reference's naive_colreduce stored in tests/golden/."""
    dev = _dev()
    for name, red, causal in golden.cases():
        q, k, scale = golden.inputs(name)
        got = _f32(q.to(dev), k.to(dev), red, causal, scale)
        assert_parity(got, golden.output(name, red, causal), red)


def test_golden_vectors_api_dtype(golden):
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    for name, red, causal in golden.cases():
        q, k, scale = golden.inputs(name)
        got = flash_colreduce(q.to(dev), k.to(dev), red, is_causal=causal, scale=scale)
        assert got.dtype == torch.float16 and got.shape == golden.output(name, red, causal).shape
        assert_parity(got, golden.output(name, red, causal), red, extra_rtol=2.0 ** -11)


# The reference's test matrix (tests/test_correctness.py:8-13): 720 cases.
@pytest.mark.parametrize("d", [16, 32, 64, 48, 72])
@pytest.mark.parametrize("m,n", [(128, 128), (131, 131), (128, 1024), (131, 1027)])
def test_reference_matrix(m, n, d):
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    for b in (1, 4, 7):
        for h in (8, 13):
            q = _rand((b, h, m, d), 0)
            k = _rand((b, h, n, d), 1)
            qd, kd = q.to(dev), k.to(dev)
            for red in ("sum", "mean", "max"):
                for causal in (False, True):
                    want = oracle_colreduce(q, k, red, causal)
                    assert_parity(_f32(qd, kd, red, causal), want, red)
                    out = flash_colreduce(qd, kd, reduction=red, is_causal=causal)
                    # the reference's own bar for the fp16 result: atol = rtol = 1e-3
                    torch.testing.assert_close(out.float().cpu(), want, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("red", ["sum", "mean", "max"])
def test_config_nonsquare_batch(red):
    """B=8, H=16, M=N=512, d=64, not causal."""
    dev = _dev()
    q, k = _rand((8, 16, 512, 64), 0), _rand((8, 16, 512, 64), 1)
    assert_parity(_f32(q.to(dev), k.to(dev), red, False), oracle_colreduce(q, k, red, False), red)


@pytest.mark.parametrize("red", ["sum", "mean", "max"])
def test_config_decode(red):
    """q (1,32,128,128), k (1,32,4096,128), right-aligned causal mask."""
    dev = _dev()
    q, k = _rand((1, 32, 128, 128), 0), _rand((1, 32, 4096, 128), 1)
    assert_parity(_f32(q.to(dev), k.to(dev), red, True), oracle_colreduce(q, k, red, True), red)


def _vlm_inputs(b, h, n, d, seed):
    """Attention-sink keys 0-3 scaled by 8; keys 512-6655 drawn with standard deviation 0.5."""
    q = _rand((b, h, n, d), seed).float()
    k = _rand((b, h, n, d), seed + 1).float()
    k[:, :, 0:4] *= 8
    k[:, :, 512:6656] *= 0.5
    return q.half(), k.half()


def test_config_vlm_pruning_heads():
    """Three heads of the B=4, H=32, M=N=8192, d=128 causal mean configuration."""
    dev = _dev()
    q, k = _vlm_inputs(1, 3, 8192, 128, 10)
    for red in ("mean", "sum", "max"):
        assert_parity(_f32(q.to(dev), k.to(dev), red, True), oracle_colreduce(q, k, red, True), red)


def test_config_vlm_pruning_whole_problem():
    """The whole B=4, H=32, M=N=8192, d=128 causal configuration: one head of every batch entry
    against the oracle (mean, the configuration's reduction), every head through properties."""
    dev = _dev()
    b, h, n, d = 4, 32, 8192, 128
    q, k = _vlm_inputs(b, h, n, d, 30)
    qd, kd = q.to(dev), k.to(dev)
    mean = _f32(qd, kd, "mean", True)
    total = _f32(qd, kd, "sum", True)
    for bi, hi in ((0, 5), (1, 13), (2, 22), (3, 31)):
        want = oracle_colreduce(q[bi:bi + 1, hi:hi + 1], k[bi:bi + 1, hi:hi + 1], "mean", True)
        assert_parity(mean[bi:bi + 1, hi:hi + 1], want, "mean")
    # every softmax row sums to one: the column sums of a head add up to its number of rows
    torch.testing.assert_close(total.double().sum(dim=-1).cpu(), torch.full((b, h), float(n), dtype=torch.float64),
                               rtol=1e-4, atol=0)
    # M == N: column j is seen by the n - j queries j .. n-1, and that is its mean divisor (flash.py:377-384)
    div = torch.arange(n, 0, -1, dtype=torch.float32, device=dev)
    torch.testing.assert_close(mean * div, total, rtol=1e-6, atol=1e-30)
    assert bool((mean > 0).all()) and bool((mean <= 1 + 1e-6).all())
    # the four sink keys take a visible share of every row's probability mass
    assert float((total[..., :4].sum(dim=-1) / n).min()) > 0.05


def test_long_context_properties():
    """M=N=131072, d=128, causal: checked through size-independent properties and row slices."""
    from flash_colreduce_b200 import colreduce_partial

    dev = _dev()
    n, d, h = 131072, 128, 2
    q, k = _rand((1, h, n, d), 20), _rand((1, h, n, d), 21)
    qd, kd = q.to(dev), k.to(dev)
    scale = 1 / math.sqrt(d)
    total = _f32(qd, kd, "sum", True)
    # every softmax row sums to one, so the column sums add up to the number of rows
    torch.testing.assert_close(total.double().sum(dim=-1).cpu(), torch.full((1, h), float(n), dtype=torch.float64),
                               rtol=1e-4, atol=0)
    again = _f32(qd, kd, "sum", True)
    assert torch.equal(total, again), "summation order must be fixed"
    mx = _f32(qd, kd, "max", True)
    assert float(mx.max()) <= 1.0 + 1e-6 and float(mx.min()) > 0.0
    assert bool((mx <= total + 1e-6).all())
    assert float(mx[..., -1].min()) == pytest.approx(float(total[..., -1].min()))  # last key: one query
    # row slices against the oracle: first rows, a slice across the middle, the last rows
    acc = torch.zeros_like(total)
    for lo, hi in ((0, 384), (65500, 65800), (n - 300, n)):
        part = colreduce_partial(qd[:, :, lo:hi], kd[:, :, :hi], "sum", True, scale, causal_offset=lo)
        want = oracle_colreduce(q, k[:, :, :hi], "sum", True, scale, row_range=(lo, hi))
        # oracle_colreduce aligns the mask for an (n x hi) problem: rows see keys <= i + max(hi - n, 0) = i
        assert_parity(part, want, "sum")
        acc[..., :hi] += part
    assert bool((acc <= total * (1 + 1e-4) + 1e-6).all())


def test_masked_positions_are_exact_zero():
    """Keys no query of a slice may attend must come out as 0.0 exactly."""
    from flash_colreduce_b200 import colreduce_partial

    dev = _dev()
    q, k = _rand((1, 2, 300, 64), 3), _rand((1, 2, 300, 64), 4)
    k[:, :, 200:] *= 30  # would dominate every softmax if the mask leaked
    for red in ("sum", "max"):
        got = colreduce_partial(q[:, :, :70].to(dev), k.to(dev), red, True, 0.125, causal_offset=0)
        assert bool((got[..., 70:] == 0).all())
        want = oracle_colreduce(q, k, red, True, 0.125, row_range=(0, 70))
        assert_parity(got, want, red)


@pytest.mark.parametrize("m,n", [(300, 100), (1000, 257), (1, 500), (129, 128)])
def test_more_queries_than_keys_and_edge_shapes(m, n):
    dev = _dev()
    q, k = _rand((2, 3, m, 64), 5), _rand((2, 3, n, 64), 6)
    for red in ("sum", "mean", "max"):
        for causal in (False, True):
            assert_parity(_f32(q.to(dev), k.to(dev), red, causal), oracle_colreduce(q, k, red, causal), red)


@pytest.mark.parametrize("b,h,m,n,d", [(1, 1, 1, 1, 8), (3, 5, 1, 7, 8), (2, 2, 7, 1, 24), (16, 64, 2, 3, 16),
                                       (1, 2, 129, 255, 120), (1, 1, 257, 129, 104), (1, 3, 640, 384, 128),
                                       (1, 2, 300, 700, 256), (2, 1, 1100, 513, 192), (1, 3, 257, 2049, 136)])
def test_degenerate_and_odd_head_dims(b, h, m, n, d):
    dev = _dev()
    q, k = _rand((b, h, m, d), 30), _rand((b, h, n, d), 31)
    for red in ("sum", "mean", "max"):
        for causal in (False, True):
            assert_parity(_f32(q.to(dev), k.to(dev), red, causal), oracle_colreduce(q, k, red, causal), red)


@pytest.mark.parametrize("d", [64, 128, 192])
def test_many_items_per_cta_with_a_skipped_half_block(d):
    """More work items than CTAs, several streamed tiles per item, and a last key block whose
    second half lies beyond N: every CTA runs items of both kinds back to back."""
    dev = _dev()
    q, k = _rand((4, 64, 300, d), 40), _rand((4, 64, 300, d), 41)
    for red in ("sum", "max"):
        for causal in (False, True):
            assert_parity(_f32(q.to(dev), k.to(dev), red, causal), oracle_colreduce(q, k, red, causal), red)


@pytest.mark.parametrize("b,h,m,n,d", [(1, 2, 1, 1024, 128), (2, 3, 7, 1500, 64), (1, 4, 64, 4099, 128),
                                       (1, 2, 100, 2048, 72), (1, 1, 128, 8192, 128), (3, 50, 33, 1027, 64),
                                       (1, 160, 128, 1024, 128), (2, 3, 50, 2048, 256), (1, 2, 9, 1100, 200)])
def test_decode_shapes_stream_the_keys(b, h, m, n, d):
    """M <= 128 with at least 8 key tiles: the key-streaming kernels (one query tile per head kept in
    shared memory, several work items and heads per CTA in the last two cases)."""
    from flash_colreduce_b200 import _native as nat

    dev = _dev()
    q, k = _rand((b, h, m, d), 50), _rand((b, h, n, d), 51)
    pr = nat.make_problem(b, h, m, n, d, q.stride(), k.stride(), nat.FCR_F16, 0, True, 0.1)
    assert nat.plan(pr, 148).key_stream == 1
    for red in ("sum", "mean", "max"):
        for causal in (False, True):
            assert_parity(_f32(q.to(dev), k.to(dev), red, causal), oracle_colreduce(q, k, red, causal), red)


def test_decode_full_size_properties():
    """A decode batch too large for the oracle (2 GiB of keys): every query row's softmax sums to one, so
    the columns of a head sum to M; max lies in (0, 1]; two runs agree bit for bit."""
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(7)
    b, h, m, n, d = 8, 32, 16, 32768, 128
    q = torch.randn(b, h, m, d, generator=g, device=dev, dtype=torch.float16)
    k = torch.randn(b, h, n, d, generator=g, device=dev, dtype=torch.float16)
    for causal in (False, True):
        s1 = flash_colreduce(q.float().half(), k, "sum", is_causal=causal).float()
        total = s1.sum(dim=-1)
        assert torch.allclose(total, torch.full_like(total, float(m)), rtol=2e-3)
        assert torch.equal(flash_colreduce(q, k, "sum", is_causal=causal).float(), s1)
        mx = flash_colreduce(q, k, "max", is_causal=causal).float()
        assert (mx > 0).all() and (mx <= 1.0 + 1e-3).all()
        # a column's mean over the queries that see it cannot exceed its max
        mean = flash_colreduce(q, k, "mean", is_causal=causal).float()
        assert (mean <= mx * (1 + 2e-3) + 1e-6).all()


def test_score_cache_is_optional():
    """M <= 16 decode: with the full workspace the columns are reduced from the cached scores, with a
    workspace that ends before the cache (plan.off_scores bytes) by a second sweep over K."""
    import ctypes as C

    from flash_colreduce_b200 import _native as nat

    dev = _dev()
    b, h, m, n, d = 2, 3, 5, 3000, 64
    q, k = _rand((b, h, m, d), 56), _rand((b, h, n, d), 57)
    qd, kd = q.to(dev), k.to(dev)
    stream = torch.cuda.current_stream().cuda_stream
    for red in ("sum", "max"):
        for causal in (False, True):
            pr = nat.make_problem(b, h, m, n, d, qd.stride(), kd.stride(), nat.FCR_F16, nat.REDUCTION_CODES[red],
                                  causal, 1 / math.sqrt(d))
            pl = nat.plan(pr, 0)
            assert pl.key_stream == 1 and pl.score_cache == 1 and 0 < pl.off_scores < pl.workspace_bytes
            want = oracle_colreduce(q, k, red, causal)
            for ws_bytes in (pl.workspace_bytes, pl.off_scores):
                ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
                out = torch.empty(b, h, n, dtype=torch.float32, device=dev)
                nat.check(nat.lib.fcr_colreduce(C.byref(pr), qd.data_ptr(), kd.data_ptr(), out.data_ptr(), nat.FCR_F32,
                                                ws.data_ptr(), ws.numel(), stream), "fcr_colreduce")
                nat.check(nat.lib.fcr_read_device_status(ws.data_ptr(), stream, None), "device status")
                assert_parity(out, want, red)
            too_small = torch.empty(pl.off_scores - 256, dtype=torch.uint8, device=dev)
            rc = nat.lib.fcr_colreduce(C.byref(pr), qd.data_ptr(), kd.data_ptr(), out.data_ptr(), nat.FCR_F32,
                                       too_small.data_ptr(), too_small.numel(), stream)
            assert rc == nat.FCR_ERR_WORKSPACE


def test_decode_shapes_other_dtypes():
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    q, k = _rand((2, 2, 40, 64), 52, torch.bfloat16), _rand((2, 2, 3000, 64), 53, torch.bfloat16)
    for red in ("sum", "max"):
        got = flash_colreduce(q.to(dev), k.to(dev), red, is_causal=True)
        assert_parity(got, oracle_colreduce(q, k, red, True), red, extra_rtol=8e-3)
    q = _tf32(_rand((1, 3, 20, 48), 54, torch.float32))
    k = _tf32(_rand((1, 3, 2500, 48), 55, torch.float32))
    for red in ("sum", "mean", "max"):
        for causal in (False, True):
            got = flash_colreduce(q.to(dev), k.to(dev), red, is_causal=causal)
            assert_parity(got, oracle_colreduce(q, k, red, causal), red)


@pytest.mark.parametrize("world,heads,m,n", [(4, 2, 1000, 1300), (8, 1, 2048, 2048), (2, 5, 300, 700), (4, 1, 100, 4096)])
def test_shards_of_several_ranks_on_one_gpu(world, heads, m, n):
    """The shard plans of a multi-GPU run (row slices with explicit mask offsets, or head ranges), executed
    rank after rank on this GPU and combined as the all-reduce would."""
    import dataclasses

    from flash_colreduce_b200 import finalize_scores
    from flash_colreduce_b200.sharding import plan_shards, sharded_colreduce

    dev = _dev()
    q, k = _rand((1, heads, m, 64), 70), _rand((1, heads, n, 64), 71)
    for red in ("sum", "mean", "max"):
        for causal in (False, True):
            acc = None
            for rank in range(world):
                spec = plan_shards(heads, m, world, rank)
                if spec.heads == 0:
                    continue
                alone = dataclasses.replace(spec, world=1)  # no collective: the partial comes back as it is
                part = sharded_colreduce(q[:, spec.head_lo:spec.head_hi].to(dev), k[:, spec.head_lo:spec.head_hi].to(dev),
                                         red, causal, spec=alone, total_heads=heads,
                                         finalize_fn=lambda a, *rest: a)
                if acc is None:
                    acc = part
                else:
                    acc = torch.maximum(acc, part) if red == "max" else acc + part
            got = finalize_scores(acc[None].contiguous(), m, red, causal, torch.float32)
            assert_parity(got, oracle_colreduce(q, k, red, causal), red)


def test_zero_scale_gives_uniform_rows():
    dev = _dev()
    q, k = _rand((1, 2, 100, 64), 32), _rand((1, 2, 300, 64), 33)
    got = _f32(q.to(dev), k.to(dev), "sum", False, 0.0)
    torch.testing.assert_close(got.cpu(), torch.full((1, 2, 300), 100.0 / 300.0), rtol=1e-5, atol=1e-6)
    assert_parity(_f32(q.to(dev), k.to(dev), "mean", True, 0.0), oracle_colreduce(q, k, "mean", True, 0.0), "mean")


def test_many_heads_and_batch_strides():
    """More work items than any one CTA sees, and a batch taken out of a larger tensor."""
    dev = _dev()
    q, k = _rand((6, 40, 130, 64), 34), _rand((6, 40, 200, 64), 35)
    qd, kd = q.to(dev), k.to(dev)
    assert_parity(_f32(qd, kd, "sum", True), oracle_colreduce(q, k, "sum", True), "sum")
    assert_parity(_f32(qd[1:5:2, 3:33], kd[1:5:2, 3:33], "mean", True),
                  oracle_colreduce(q[1:5:2, 3:33], k[1:5:2, 3:33], "mean", True), "mean")


@pytest.mark.parametrize("scale", [0.3, -0.2, 1.5])
def test_user_scale(scale):
    dev = _dev()
    q, k = _rand((1, 2, 200, 32), 7), _rand((1, 2, 333, 32), 8)
    for red in ("sum", "max"):
        assert_parity(_f32(q.to(dev), k.to(dev), red, True, scale), oracle_colreduce(q, k, red, True, scale), red)


def test_bfloat16_inputs():
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    q, k = _rand((1, 2, 260, 128), 9, torch.bfloat16), _rand((1, 2, 400, 128), 10, torch.bfloat16)
    for red in ("sum", "mean", "max"):
        want = oracle_colreduce(q, k, red, True)
        assert_parity(_f32(q.to(dev), k.to(dev), red, True), want, red)
        out = flash_colreduce(q.to(dev), k.to(dev), red, is_causal=True)
        assert out.dtype == torch.bfloat16
        assert_parity(out, want, red, extra_rtol=2.0 ** -8)


def test_strided_and_odd_inputs():
    """Row slices, (B,M,H,D) storage, and a head dimension that is not a multiple of 8."""
    dev = _dev()
    q, k = _rand((2, 4, 500, 64), 11), _rand((2, 4, 700, 64), 12)
    qd, kd = q.to(dev), k.to(dev)
    got = _f32(qd[:, :, 100:400], kd, "sum", False)
    assert_parity(got, oracle_colreduce(q[:, :, 100:400], k, "sum", False), "sum")
    q_bmhd = qd.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)  # logical (B,H,M,D), memory (B,M,H,D)
    assert not q_bmhd.is_contiguous()
    assert_parity(_f32(q_bmhd, kd, "mean", True), oracle_colreduce(q, k, "mean", True), "mean")
    q2, k2 = _rand((1, 2, 150, 20), 13), _rand((1, 2, 90, 20), 14)
    assert_parity(_f32(q2.to(dev), k2.to(dev), "max", True), oracle_colreduce(q2, k2, "max", True), "max")


def test_errors_match_the_reference_messages():
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    q = torch.zeros(1, 2, 8, 16, dtype=torch.float16, device=dev)
    with pytest.raises(ValueError, match="must be on CUDA device"):
        flash_colreduce(q.cpu(), q, "sum")
    with pytest.raises(ValueError, match="same batch size, number of heads, and head dimension"):
        flash_colreduce(q, torch.zeros(1, 3, 8, 16, dtype=torch.float16, device=dev), "sum")
    with pytest.raises(ValueError, match="Invalid reduction: prod"):
        flash_colreduce(q, q, "prod")
    with pytest.raises(TypeError):
        flash_colreduce(q.double(), q.double(), "sum")
    with pytest.raises(TypeError):
        flash_colreduce(q, q.float(), "sum")
    with pytest.raises(ValueError, match="exceeds 128"):
        flash_colreduce(torch.zeros(1, 1, 8, 136, device=dev), torch.zeros(1, 1, 8, 136, device=dev), "sum")
    assert flash_colreduce(q[:, :, :0], q, "sum").shape == (1, 2, 8)
    assert flash_colreduce(q, q[:, :, :0], "sum").shape == (1, 2, 0)


def test_runs_on_the_current_stream_without_sync():
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    q, k = _rand((1, 4, 512, 64), 15).to(dev), _rand((1, 4, 512, 64), 16).to(dev)
    base = flash_colreduce(q, k, "sum")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        other = flash_colreduce(q, k, "sum")
    s.synchronize()
    assert torch.equal(base, other)


def test_capturable_in_a_cuda_graph():
    """The whole call (memset + kernels, no host sync) can be captured once and replayed."""
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    q, k = _rand((2, 4, 300, 64), 40).to(dev), _rand((2, 4, 700, 64), 41).to(dev)
    os.environ["FCR_DEBUG_SYNC"] = "0"  # the status read-back synchronises, which a capture forbids
    try:
        eager = flash_colreduce(q, k, "mean", is_causal=True)  # also performs the one-time kernel set-up
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = flash_colreduce(q, k, "mean", is_causal=True)
        q2 = _rand((2, 4, 300, 64), 42).to(dev)
        q.copy_(q2)  # new inputs in the captured buffers
        graph.replay()
        torch.cuda.synchronize()
    finally:
        os.environ["FCR_DEBUG_SYNC"] = "1"
    want = flash_colreduce(q, k, "mean", is_causal=True)
    assert torch.equal(captured, want)
    assert not torch.equal(captured, eager)


def test_decode_and_selection_capturable_in_a_cuda_graph():
    """Same for a decode shape (key-streaming kernels, score cache) followed by the top-k selection."""
    from flash_colreduce_b200 import flash_colreduce_topk

    dev = _dev()
    q, k = _rand((1, 6, 4, 64), 43).to(dev), _rand((1, 6, 2000, 64), 44).to(dev)
    os.environ["FCR_DEBUG_SYNC"] = "0"
    try:
        flash_colreduce_topk(q, k, "sum", 100, is_causal=True)  # one-time kernel set-up outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            vals, idx = flash_colreduce_topk(q, k, "sum", 100, is_causal=True)
        q.copy_(_rand((1, 6, 4, 64), 45).to(dev))
        graph.replay()
        torch.cuda.synchronize()
    finally:
        os.environ["FCR_DEBUG_SYNC"] = "1"
    want_vals, want_idx = flash_colreduce_topk(q, k, "sum", 100, is_causal=True)
    assert torch.equal(idx, want_idx) and torch.equal(vals, want_vals)


def test_host_resident_inputs():
    """flash_colreduce_host streams head groups through the GPU; result equals the device API's."""
    from flash_colreduce_b200 import flash_colreduce, flash_colreduce_host

    dev = _dev()
    q, k = _rand((2, 6, 400, 64), 50), _rand((2, 6, 900, 64), 51)
    want = oracle_colreduce(q, k, "mean", True)
    for pinned in (False, True):
        qh = q.pin_memory() if pinned else q
        kh = k.pin_memory() if pinned else k
        for group in (None, 1, 4, 6):
            got = flash_colreduce_host(qh, kh, "mean", is_causal=True, device=dev, group_heads=group)
            assert not got.is_cuda and got.shape == (2, 6, 900) and got.dtype == torch.float16
            assert_parity(got, want, "mean", extra_rtol=2.0 ** -11)
            assert torch.equal(got, flash_colreduce(q.to(dev), k.to(dev), "mean", is_causal=True).cpu())
    with pytest.raises(ValueError, match="host tensors"):
        flash_colreduce_host(q.to(dev), k.to(dev), "sum")
    with pytest.raises(ValueError, match="Invalid reduction"):
        flash_colreduce_host(q, k, "prod")


def _tf32(x: torch.Tensor) -> torch.Tensor:
    """fp32 values with the 13 low mantissa bits cleared: exactly representable as TF32."""
    return (x.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32)


@pytest.mark.parametrize("d", [16, 32, 40, 64, 96, 128])
def test_float32_inputs_run_as_tf32(d):
    """fp32 tensors (the reference multiplies them as TF32 in tl.dot, flash.py:59) against the oracle
    on the same TF32-representable values; the result dtype is fp32."""
    from flash_colreduce_b200 import flash_colreduce

    dev = _dev()
    q = _tf32(_rand((2, 3, 300, d), 60, torch.float32))
    k = _tf32(_rand((2, 3, 500, d), 61, torch.float32))
    for red in ("sum", "mean", "max"):
        for causal in (False, True):
            got = flash_colreduce(q.to(dev), k.to(dev), red, is_causal=causal)
            assert got.dtype == torch.float32
            assert_parity(got, oracle_colreduce(q, k, red, causal), red)
