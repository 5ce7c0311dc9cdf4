import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN_PATH = os.path.join(ROOT, "tests", "golden", "naive_golden.npz")


def _ensure_library_built():
    """Builds the sm_100a library in-tree when it is missing or older than its sources (nvcc cross-compiles)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("_fcr_build", os.path.join(ROOT, "flash_colreduce_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


_ensure_library_built()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


class Golden:
    """Inputs and reference outputs written by tests/golden/make_golden.py."""

    def __init__(self):
        self.data = np.load(GOLDEN_PATH)
        self.names = sorted({key.split("__")[1] for key in self.data.files if key.startswith("in__")})

    def inputs(self, name):
        q = torch.from_numpy(self.data[f"in__{name}__q"])
        k = torch.from_numpy(self.data[f"in__{name}__k"])
        s = float(self.data[f"in__{name}__scale"])
        return q, k, (None if s < 0 else s)

    def cases(self):
        """Yields (name, reduction, is_causal)."""
        for key in sorted(self.data.files):
            if key.startswith("out__"):
                _, name, red, causal = key.split("__")
                yield name, red, bool(int(causal))

    def output(self, name, reduction, is_causal):
        return torch.from_numpy(self.data[f"out__{name}__{reduction}__{int(is_causal)}"])


@pytest.fixture(scope="session")
def golden():
    return Golden()


def assert_parity(got: torch.Tensor, want: torch.Tensor, reduction: str, extra_rtol: float = 0.0):
    """The parity bar of the operator: sum / mean within rtol 2e-3, atol 1e-5; max within 1e-3.

    ``extra_rtol`` widens the relative bound by the rounding of a 16-bit output
    dtype (2^-11 for fp16, 2^-8 for bf16) when the result is not fp32.
    """
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    assert got.shape == want.shape
    assert not torch.isnan(got).any()
    if reduction == "max":
        bound = 1e-3 + extra_rtol * want.abs()
    else:
        bound = 1e-5 + (2e-3 + extra_rtol) * want.abs()
    err = (got - want).abs()
    worst = (err / bound).max().item()
    assert worst <= 1.0, f"parity violated: worst error/bound = {worst:.3f}, max abs err {err.max().item():.3e}"
