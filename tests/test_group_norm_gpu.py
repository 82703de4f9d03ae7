"""Parity of the CUDA GroupNorm path (through the C ABI) against the golden vectors and the FP64
oracle on the same seeded inputs; tolerances of the reference's tests
(tests/test_native_group_norm.py:36,42 of the reference) or tighter."""
import numpy as np
import pytest

import b200conv
from golden_cases import gn_case_id, group_norm_cases
from oracle import group_norm_oracle as gn
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-5   # max relative L2 error against the FP64 oracle


def _f32(v):
    return None if v is None else np.asarray(v, np.float32)


@pytest.mark.parametrize("c", group_norm_cases(), ids=gn_case_id)
def test_golden_cases(c):
    x, g, w, b = _f32(c["x"]), _f32(c["g"]), _f32(c["w"]), _f32(c["b"])
    y, mean, rstd = b200conv.group_norm_forward(x, c["groups"], w, b, 1e-5)
    np.testing.assert_allclose(y, c["y"], rtol=5e-4, atol=4e-5)
    np.testing.assert_allclose(mean, c["mean"], rtol=5e-4, atol=4e-5)
    np.testing.assert_allclose(rstd, c["rstd"], rtol=5e-4, atol=4e-5)
    dx, dw, db = b200conv.group_norm_backward(g, x, mean, rstd, c["groups"], w)
    for got, want in ((dx, c["dx"]), (dw, c["dw"]), (db, c["db"])):
        np.testing.assert_allclose(got, want, rtol=8e-4, atol=7e-5)


# planes longer than one segment, planes off the vector width, one channel per group, one group,
# many channels per group, a single value per plane, U-Net sized blocks
SHAPES = [((2, 32, 64, 64), 8), ((3, 6, 50, 50), 2), ((2, 12, 33, 31), 3), ((4, 16, 8, 8), 16), ((2, 24, 16, 16), 1),
          ((5, 64, 7, 7), 4), ((3, 40), 5), ((2, 8, 5000), 2), ((1, 320, 16, 16), 32), ((2, 6, 3, 100, 50), 3),
          ((80, 128, 32, 32), 8), ((50, 384, 28, 28), 12), ((3, 32, 56, 56), 4)]


@pytest.mark.parametrize("shape,groups", SHAPES, ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else f"g{v}")
@pytest.mark.parametrize("affine", [False, True], ids=["plain", "affine"])
def test_against_the_fp64_oracle(shape, groups, affine):
    rng = np.random.default_rng(sum(shape) + groups)
    c = shape[1]
    x = (rng.standard_normal(shape) * 1.5 + 0.7).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    w = rng.standard_normal(c).astype(np.float32) if affine else None
    b = rng.standard_normal(c).astype(np.float32) if affine else None
    y, mean, rstd = b200conv.group_norm_forward(x, groups, w, b, 1e-5)
    # blocks of 50 KB to 100 KB with planes of whole 16-byte groups stay resident in shared memory once
    # there are four of them or more per SM
    block_bytes, hw = 4 * x[0].size // groups, x[0, 0].size
    resident = hw % 4 == 0 and 50 * 1024 < block_bytes <= 100 * 1024 and shape[0] * groups >= 4 * b200conv.lib().b200_device_sm_count()
    assert b200conv.last_kernel() == ("gn_forward_bulk" if resident else "gn_forward")
    assert b200conv.device_status() == 0
    wy, wmean, wrstd = gn.forward(x, groups, w, b, 1e-5, dtype=np.float64)
    assert oracle.rel_l2(y, wy) <= GATE
    np.testing.assert_allclose(mean, wmean, rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(rstd, wrstd, rtol=5e-6)
    dx, dw, db = b200conv.group_norm_backward(g, x, mean, rstd, groups, w)
    wdx, wdw, wdb = gn.backward(g, x, mean, rstd, groups, w, dtype=np.float64)
    assert oracle.rel_l2(dx, wdx) <= 2 * GATE
    assert oracle.rel_l2(dw, wdw) <= 2 * GATE
    assert oracle.rel_l2(db, wdb) <= 2 * GATE


@pytest.mark.parametrize("mask", [(True, False, False), (False, True, False), (False, False, True), (True, True, True),
                                  (False, False, False)])
def test_output_masks(mask):
    rng = np.random.default_rng(123)
    x, g, w = rng.standard_normal((2, 8, 5, 6)).astype(np.float32), rng.standard_normal((2, 8, 5, 6)).astype(np.float32), \
        rng.standard_normal(8).astype(np.float32)
    _, mean, rstd = b200conv.group_norm_forward(x, 4, w, None, 1e-5)
    got = b200conv.group_norm_backward(g, x, mean, rstd, 4, w, mask=mask)
    want = gn.backward(g, x, mean, rstd, 4, w, dtype=np.float64)
    for yes, a, e in zip(mask, got, want):
        if yes:
            np.testing.assert_allclose(a, e, rtol=8e-4, atol=7e-5)
        else:
            assert a is None


def test_large_offset_keeps_the_variance():
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((2, 8, 40, 40)) * 0.1 + 10000.0).astype(np.float32)
    y, mean, rstd = b200conv.group_norm_forward(x, 2, None, None, 1e-5)
    wy, wmean, wrstd = gn.forward(x, 2, None, None, 1e-5, dtype=np.float64)
    np.testing.assert_allclose(rstd, wrstd, rtol=3e-5)
    np.testing.assert_allclose(mean, wmean, rtol=0, atol=1e-3)
    np.testing.assert_allclose(y, wy, rtol=3e-4, atol=0.008)


def test_full_size_block_properties():
    # 16 x 256 x 64 x 64 with 32 groups (a diffusion U-Net block, 67 MB): every (sample, group) block
    # of y has zero mean and unit variance; dx is orthogonal to 1 and to the normalised input
    rng = np.random.default_rng(9)
    shape, groups = (16, 256, 64, 64), 32
    x = rng.standard_normal(shape, dtype=np.float32) * 3.0 - 1.0
    g = rng.standard_normal(shape, dtype=np.float32)
    y, mean, rstd = b200conv.group_norm_forward(x, groups, None, None, 1e-5)
    blocks = y.reshape(16, groups, -1).astype(np.float64)
    assert np.abs(blocks.mean(axis=2)).max() < 1e-5
    np.testing.assert_allclose(blocks.var(axis=2), 1.0, rtol=1e-4)
    dx, dw, db = b200conv.group_norm_backward(g, x, mean, rstd, groups, None)
    dblocks = dx.reshape(16, groups, -1).astype(np.float64)
    scale = np.abs(dblocks).sum(axis=2)
    assert (np.abs(dblocks.sum(axis=2)) / scale).max() < 1e-5
    assert (np.abs((dblocks * blocks).sum(axis=2)) / scale).max() < 1e-5
    wdx, wdw, wdb = gn.backward(g, x, mean, rstd, groups, None, dtype=np.float64)
    assert oracle.rel_l2(dx, wdx) <= 2 * GATE
    assert oracle.rel_l2(dw, wdw) <= 1e-4 and oracle.rel_l2(db, wdb) <= 1e-4


def test_invalid_arguments():
    b200conv.init()
    assert b200conv.lib().b200_group_norm_workspace(2, 6, 4, 4) == 0   # channels not divisible by groups
    with pytest.raises(b200conv.B200Error, match="invalid batch, channel, group or spatial"):
        b200conv.group_norm_forward(np.zeros((2, 6, 4), np.float32), 4)
    with pytest.raises(ValueError, match="shape mismatch"):
        b200conv.group_norm_backward(np.zeros((2, 4, 4), np.float32), np.zeros((2, 4, 5), np.float32),
                                     np.zeros((2, 2), np.float32), np.ones((2, 2), np.float32), 2)
