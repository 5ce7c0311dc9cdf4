"""The oracle against the reference's outputs, a closed form and the C restatement (CPU only)."""
import math

import numpy as np
import pytest
import torch

from oracle import oracle_colreduce, oracle_valid_scores
from oracle.build_oracle import colreduce_ref


def test_golden_file_is_complete(golden):
    cases = list(golden.cases())
    assert len(cases) == 43
    assert "c1" in golden.names


def test_python_oracle_matches_reference_outputs(golden):
    for name, red, causal in golden.cases():
        q, k, scale = golden.inputs(name)
        got = oracle_colreduce(q, k, red, causal, scale, compute_dtype=torch.float32)
        want = golden.output(name, red, causal)
        torch.testing.assert_close(got, want, rtol=2e-5, atol=1e-7, msg=lambda m: f"{name} {red} {causal}: {m}")


def test_python_oracle_blocking_is_exact_enough(golden):
    q, k, scale = golden.inputs("dec131_d16")
    for red in ("sum", "mean", "max"):
        a = oracle_colreduce(q, k, red, True, scale, compute_dtype=torch.float64, block_rows=7)
        b = oracle_colreduce(q, k, red, True, scale, compute_dtype=torch.float64, block_rows=4096)
        torch.testing.assert_close(a, b, rtol=1e-12, atol=1e-14)


def test_c_oracle_matches_reference_outputs(golden):
    for name, red, causal in golden.cases():
        q, k, scale = golden.inputs(name)
        s = 1 / math.sqrt(q.shape[-1]) if scale is None else scale
        got = colreduce_ref(q.float().numpy(), k.float().numpy(), red, causal, s)
        want = golden.output(name, red, causal).numpy()
        np.testing.assert_allclose(got, want, rtol=3e-5, atol=2e-7, err_msg=f"{name} {red} {causal}")


def test_row_range_and_partial_mean():
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, 2, 50, 8, generator=g)
    k = torch.randn(1, 2, 90, 8, generator=g)
    full = oracle_colreduce(q, k, "sum", True, compute_dtype=torch.float64)
    parts = sum(oracle_colreduce(q, k, "sum", True, compute_dtype=torch.float64, row_range=(lo, lo + 10))
                for lo in range(0, 50, 10))
    torch.testing.assert_close(parts, full, rtol=1e-12, atol=1e-14)
    mean = oracle_colreduce(q, k, "mean", True, compute_dtype=torch.float64)
    unnorm = oracle_colreduce(q, k, "mean", True, compute_dtype=torch.float64, apply_mean=False)
    torch.testing.assert_close(unnorm, full)
    c = 40
    div = torch.cat([torch.full((c,), 50.0), torch.arange(50, 0, -1).double()])
    torch.testing.assert_close(mean, full / div)


@pytest.mark.parametrize("m,n", [(5, 5), (4, 9), (9, 4)])
def test_closed_form_equal_keys(m, n):
    """All keys equal => uniform softmax over the visible keys => column sum_i 1/valid(i)."""
    q = torch.randn(1, 1, m, 4, generator=torch.Generator().manual_seed(3))
    k = torch.ones(1, 1, n, 4)
    c = max(n - m, 0)
    valid = [min(i + c + 1, n) for i in range(m)]
    want_sum = torch.tensor([sum(1.0 / valid[i] for i in range(m) if j < valid[i]) for j in range(n)], dtype=torch.float64)
    want_max = torch.tensor([max((1.0 / valid[i] for i in range(m) if j < valid[i]), default=0.0) for j in range(n)],
                            dtype=torch.float64)
    got_sum = oracle_colreduce(q, k, "sum", True, compute_dtype=torch.float64)[0, 0]
    got_max = oracle_colreduce(q, k, "max", True, compute_dtype=torch.float64)[0, 0]
    torch.testing.assert_close(got_sum, want_sum, rtol=1e-12, atol=1e-14)
    torch.testing.assert_close(got_max, want_max, rtol=1e-12, atol=1e-14)
    assert oracle_valid_scores(1, 1, m, n, True) == sum(valid)
    nc = oracle_colreduce(q, k, "mean", False, compute_dtype=torch.float64)[0, 0]
    torch.testing.assert_close(nc, torch.full((n,), 1.0 / n, dtype=torch.float64), rtol=1e-12, atol=1e-14)


def test_invalid_reduction():
    q = torch.zeros(1, 1, 2, 2)
    with pytest.raises(ValueError, match="Invalid reduction"):
        oracle_colreduce(q, q, "prod")
