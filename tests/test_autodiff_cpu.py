"""The oracle against the known-answer gradients of helium/tests/autodiff.rs (graphs in autodiff_cases.py)."""
import numpy as np
import pytest

from autodiff_cases import cases
from helpers import O


@pytest.mark.parametrize("case", cases(), ids=lambda c: c[0])
def test_oracle_reproduces_reference_gradients(case):
    name, where, g, ins, want = case
    got = O.evaluate(g, ins)
    for o, a, b in zip(g.outputs, got, want):
        # the reference compares with assert_ulps_eq! (4 ulps by default) or assert_eq!
        assert np.allclose(np.asarray(a, dtype=np.float64).reshape(-1), np.asarray(b, dtype=np.float64).reshape(-1), rtol=5e-7, atol=0), (name, where, a, b)
