"""Pins the GroupNorm oracle against the golden vectors (PyTorch CPU FP64 on the reference's seeded
cases) with the tolerances of the reference's tests (tests/test_native_group_norm.py:36,42 there)."""
import numpy as np
import pytest

from golden_cases import gn_case_id, group_norm_cases
from oracle import group_norm_oracle as gn

CASES = group_norm_cases()


def _run(c, dtype):
    y, mean, rstd = gn.forward(c["x"], c["groups"], c["w"], c["b"], 1e-5, dtype)
    dx, dw, db = gn.backward(c["g"], c["x"], mean, rstd, c["groups"], c["w"], dtype=dtype)
    return dict(y=y, mean=mean, rstd=rstd, dx=dx, dw=dw, db=db)


@pytest.mark.parametrize("c", CASES, ids=gn_case_id)
def test_fp64_oracle_matches_golden_tightly(c):
    got = _run(c, np.float64)
    for k, v in got.items():
        np.testing.assert_allclose(v, c[k], rtol=1e-9, atol=1e-9, err_msg=k)


@pytest.mark.parametrize("c", CASES, ids=gn_case_id)
def test_fp32_oracle_matches_golden_within_the_reference_tolerances(c):
    got = _run(c, np.float32)
    np.testing.assert_allclose(got["y"], c["y"], rtol=5e-4, atol=4e-5)
    for k in ("mean", "rstd"):
        np.testing.assert_allclose(got[k], c[k], rtol=5e-4, atol=4e-5)
    for k in ("dx", "dw", "db"):
        np.testing.assert_allclose(got[k], c[k], rtol=8e-4, atol=7e-5, err_msg=k)
