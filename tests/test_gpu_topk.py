"""Top-k selection over the column scores (fcr_topk), against torch.topk on the CPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _check(scores_cpu: torch.Tensor, k: int):
    from flash_colreduce_b200 import topk_columns

    vals, idx = topk_columns(scores_cpu.to(_dev()), k)
    vals, idx = vals.cpu(), idx.cpu()
    assert idx.shape == scores_cpu.shape[:-1] + (k,) and idx.dtype == torch.int64
    # positions ascending and distinct, values are the scores at those positions
    assert (idx[..., 1:] > idx[..., :-1]).all()
    assert torch.equal(vals, torch.gather(scores_cpu, -1, idx))
    # the same multiset of values as torch.topk ...
    want_vals, _ = torch.topk(scores_cpu.float(), k, dim=-1)
    got_sorted = vals.float().sort(dim=-1, descending=True)[0]
    assert torch.equal(got_sorted, want_vals)
    # ... and among the scores equal to the k-th largest, the lowest positions
    flat, fidx = scores_cpu.float().reshape(-1, scores_cpu.shape[-1]), idx.reshape(-1, k)
    for r in range(min(flat.shape[0], 16)):
        thr = want_vals.reshape(-1, k)[r, -1]
        want = torch.cat([(flat[r] > thr).nonzero().flatten(),
                          (flat[r] == thr).nonzero().flatten()[: k - int((flat[r] > thr).sum())]]).sort()[0]
        assert torch.equal(fidx[r], want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,n,k", [(1, 1, 1), (3, 100, 7), (5, 4096, 4096), (2, 5000, 1), (4, 70001, 2500),
                                      (300, 1027, 257), (3, 200003, 50000), (16, 131072, 1000), (40, 65536, 65536),
                                      (600, 576, 144), (1000, 2048, 2048), (400, 4096, 1), (2000, 9, 3)])
def test_matches_torch_topk(dtype, rows, n, k):
    g = torch.Generator().manual_seed(rows * 31 + n + k)
    _check(torch.rand(rows, n, generator=g).to(dtype), k)  # 16-bit dtypes: many exact ties


def test_ties_negative_values_and_infinities():
    s = torch.zeros(2, 3, 1000)
    _check(s, 10)  # all equal: the first ten positions
    s = -torch.rand(2, 3, 1000, generator=torch.Generator().manual_seed(1))
    s[0, 0, 5] = float("inf")
    s[0, 1, 7] = float("-inf")
    s[1, 2, 999] = 0.0
    _check(s, 3)
    _check(s, 999)


def test_on_the_scores_of_the_operator_and_argument_checks():
    from flash_colreduce_b200 import flash_colreduce, flash_colreduce_topk, topk_columns

    dev = _dev()
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, 4, 200, 64, generator=g).half().to(dev)
    k = torch.randn(2, 4, 700, 64, generator=g).half().to(dev)
    vals, idx = flash_colreduce_topk(q, k, "mean", 50, is_causal=True)
    scores = flash_colreduce(q, k, "mean", is_causal=True)
    assert idx.shape == (2, 4, 50) and torch.equal(vals, torch.gather(scores, -1, idx))
    _check(scores.cpu(), 50)
    none_vals, idx2 = topk_columns(scores, 50, return_values=False)
    assert none_vals is None and torch.equal(idx2, idx)
    with pytest.raises(ValueError, match="must lie in"):
        topk_columns(scores, 0)
    with pytest.raises(ValueError, match="must lie in"):
        topk_columns(scores, 701)
    with pytest.raises(TypeError):
        topk_columns(scores.double(), 3)
    with pytest.raises(ValueError, match="CUDA"):
        topk_columns(scores.cpu(), 3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,n", [(1, 1), (3, 100), (7, 8192), (2, 70001), (500, 600)])
def test_threshold_selection(dtype, rows, n):
    from flash_colreduce_b200 import select_columns

    g = torch.Generator().manual_seed(rows + n)
    s = torch.rand(rows, n, generator=g).to(dtype)
    for thr in (-1.0, 0.25, 0.9, 2.0):
        idx, cnt = select_columns(s.to(_dev()), thr)
        idx, cnt = idx.cpu(), cnt.cpu()
        assert idx.shape == (rows, n) and cnt.shape == (rows,)
        for r in range(min(rows, 8)):
            want = (s[r].float() > thr).nonzero().flatten()
            assert cnt[r].item() == want.numel()
            assert torch.equal(idx[r, : want.numel()], want)


@pytest.mark.parametrize("rows_shape,n,k", [((2, 300), 576, 144), ((1, 1000), 2048, 2048)])
def test_many_short_rows_on_a_side_stream_right_after_the_operator(rows_shape, n, k):
    """The 256-thread launch shape (at least two rows per SM) must run on the caller's stream: the
    scores are produced on a non-blocking side stream immediately before the selection reads them."""
    from flash_colreduce_b200 import flash_colreduce, topk_columns

    dev = _dev()
    b, h = rows_shape
    g = torch.Generator().manual_seed(n + k)
    q = torch.randn(b, h, 96, 64, generator=g).half().to(dev)
    key = torch.randn(b, h, n, 64, generator=g).half().to(dev)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        for _ in range(3):  # a few calls in a row keep the stream busy ahead of the selection
            scores = flash_colreduce(q, key, "sum", is_causal=True)
        vals, idx = topk_columns(scores, k)
    side.synchronize()
    scores_cpu, vals, idx = scores.cpu(), vals.cpu(), idx.cpu()
    assert torch.equal(vals, torch.gather(scores_cpu, -1, idx))
    want_vals, _ = torch.topk(scores_cpu.float(), k, dim=-1)
    assert torch.equal(vals.float().sort(dim=-1, descending=True)[0], want_vals)


def test_many_short_rows_inside_a_cuda_graph(monkeypatch):
    """Graph capture records only launches made on the capturing stream: rows >= 2 x SMs takes the
    256-thread launch shape, which has to be captured with the operator that feeds it."""
    from flash_colreduce_b200 import flash_colreduce, topk_columns

    monkeypatch.setenv("FCR_DEBUG_SYNC", "0")  # the status read-back synchronises, which a capture forbids
    dev = _dev()
    g = torch.Generator().manual_seed(11)
    q = torch.randn(2, 200, 64, 64, generator=g).half().to(dev)
    key = torch.randn(2, 200, 576, 64, generator=g).half().to(dev)
    flash_colreduce(q, key, "sum")  # first call outside the capture (one-time attribute set-up)
    topk_columns(flash_colreduce(q, key, "sum"), 144)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        scores = flash_colreduce(q, key, "sum")
        vals, idx = topk_columns(scores, 144)
    q.copy_(torch.randn(q.shape, generator=g).half())  # new inputs: the replay must see them
    graph.replay()
    torch.cuda.synchronize()
    scores_cpu = scores.cpu()
    assert torch.equal(vals.cpu(), torch.gather(scores_cpu, -1, idx.cpu()))
    want_vals, _ = torch.topk(scores_cpu.float(), 144, dim=-1)
    assert torch.equal(vals.cpu().float().sort(dim=-1, descending=True)[0], want_vals)
    fresh = flash_colreduce(q, key, "sum")
    assert torch.equal(fresh.cpu(), scores_cpu)
