"""Host-side behaviour of the Python API that needs no GPU."""
import pytest
import torch

import flash_colreduce_b200 as fc
from oracle import oracle_colreduce, oracle_valid_scores


def test_exports_match_the_reference_package():
    for name in ("flash_colreduce", "naive_colreduce", "__version__"):
        assert hasattr(fc, name)


def test_cpu_tensors_are_rejected_like_the_reference():
    q = torch.zeros(1, 1, 4, 8, dtype=torch.float16)
    with pytest.raises(ValueError, match="Query and key tensors must be on CUDA device."):
        fc.flash_colreduce(q, q, "sum")


def test_no_cpu_fallback_exists():
    import inspect

    from flash_colreduce_b200 import op

    src = inspect.getsource(op)
    assert "oracle" not in src and "naive_colreduce" not in src


@pytest.mark.parametrize("m,n", [(5, 5), (4, 9), (9, 4), (128, 1024)])
def test_valid_scores(m, n):
    assert fc.valid_scores(2, 3, m, n, True) == oracle_valid_scores(2, 3, m, n, True)
    assert fc.valid_scores(2, 3, m, n, False) == 6 * m * n


@pytest.mark.parametrize("red", ["sum", "mean", "max"])
@pytest.mark.parametrize("causal", [False, True])
def test_dense_definition_matches_oracle(red, causal):
    g = torch.Generator().manual_seed(2)
    q = torch.randn(2, 2, 37, 8, generator=g)
    k = torch.randn(2, 2, 53, 8, generator=g)
    got = fc.naive_colreduce(q, k, red, causal, block_rows=10)
    torch.testing.assert_close(got, oracle_colreduce(q, k, red, causal), rtol=1e-5, atol=1e-7)
    with pytest.raises(ValueError, match="Invalid reduction"):
        fc.naive_colreduce(q, k, "prod")


def test_signature_is_the_reference_operator_signature():
    """flash_colreduce(query, key, reduction, is_causal=False, scale=None), flash_colreduce/flash.py:311-317."""
    import inspect

    params = inspect.signature(fc.flash_colreduce).parameters
    assert list(params) == ["query", "key", "reduction", "is_causal", "scale"]
    assert params["is_causal"].default is False and params["scale"].default is None
    assert all(p.kind is inspect.Parameter.POSITIONAL_OR_KEYWORD for p in params.values())
    naive = inspect.signature(fc.naive_colreduce).parameters
    assert list(naive)[:5] == ["query", "key", "reduction", "is_causal", "scale"]  # naive.py:8-14
