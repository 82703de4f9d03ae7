"""Pins the BatchNorm oracle against the golden vectors (PyTorch CPU FP64 on the reference's
seeded cases) with the tolerances the reference's own tests use (tests/test_batch_norm.py:46,
:125-141 of the reference)."""
import numpy as np
import pytest

from golden_cases import batch_norm_cases, bn_case_id
from oracle import batch_norm_oracle as bn

CASES = batch_norm_cases()


def _run(c, dtype):
    y, mean, inv, rm, rv = bn.forward(c["x"], c["w"], c["b"], c["rm"], c["rv"], c["training"], c["momentum"], c["eps"], dtype)
    stats = (mean, inv) if c["training"] else (c["rm"], c["rv"])
    dx, dw, db = bn.backward(c["g"], c["x"], c["w"], *stats, c["training"], c["eps"], dtype=dtype)
    return dict(y=y, mean=mean, inv=inv, dx=dx, dw=dw, db=db, rm_out=rm, rv_out=rv)


@pytest.mark.parametrize("c", CASES, ids=bn_case_id)
def test_fp64_oracle_matches_golden_tightly(c):
    got = _run(c, np.float64)
    for k in ("y", "dx", "dw", "db", "rm_out", "rv_out") + (("mean", "inv") if c["training"] else ()):
        if c[k] is None:
            assert got[k] is None
            continue
        scale = max(1.0, float(np.nanmax(np.abs(c[k])))) if c[k].size else 1.0
        np.testing.assert_allclose(got[k], c[k], rtol=1e-9, atol=1e-9 * scale, equal_nan=True, err_msg=k)
    if not c["training"]:
        assert got["mean"].size == 0 and got["inv"].size == 0


@pytest.mark.parametrize("c", CASES, ids=bn_case_id)
def test_fp32_oracle_matches_golden_within_the_reference_tolerances(c):
    got = _run(c, np.float32)
    np.testing.assert_allclose(got["y"], c["y"], rtol=3e-4, atol=0.008 if c["tag"] == "precision" else 3e-5)
    if c["training"]:
        np.testing.assert_allclose(got["mean"], c["mean"], rtol=3e-4, atol=1e-3)
        np.testing.assert_allclose(got["inv"], c["inv"], rtol=4e-5, atol=2e-5)
    for k in ("dx", "dw", "db"):
        np.testing.assert_allclose(got[k], c[k], rtol=3e-4, atol=1e-4, err_msg=k)
    for k in ("rm_out", "rv_out"):
        if c[k] is not None:
            np.testing.assert_allclose(got[k], c[k], rtol=3e-4, atol=1e-3, equal_nan=True, err_msg=k)


def test_pair_derivative_is_antisymmetric_and_single_sample_gives_nan_variance():
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((2, 3)) * 0.1 + 10000).astype(np.float32)
    g = rng.standard_normal((2, 3)).astype(np.float32)
    _, mean, inv, _, _ = bn.forward(x, training=True, eps=1e-5)
    dx, _, _ = bn.backward(g, x, None, mean, inv, True, 1e-5)
    np.testing.assert_array_equal(dx[0], -dx[1])
    # one value per channel: variance 0, unbiased estimate 0/0 (tests/test_batch_norm.py:91-100 of the reference)
    y, _, _, _, rv = bn.forward(np.ones((1, 3), np.float32), None, None, np.zeros(3, np.float32), np.ones(3, np.float32),
                                True, .1, 1e-5)
    assert np.isnan(rv).all() and (y == 0).all()
