"""Parity of the CUDA BatchNorm path (through the C ABI) against the golden vectors and the FP64
oracle on the same seeded inputs.  Tolerances are those of the reference's own tests
(tests/test_batch_norm.py:46 and :125-141 of the reference) or tighter."""
import numpy as np
import pytest

import b200conv
from golden_cases import batch_norm_cases, bn_case_id
from oracle import batch_norm_oracle as bn
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-5   # max relative L2 error against the FP64 oracle on well-conditioned inputs


def _strided(v):
    """The vector as every other element of a longer buffer with an offset (the reference's `slice` layout)."""
    if v is None:
        return None
    store = np.zeros(2 * v.size + 3, np.float32)
    store[1:1 + 2 * v.size:2] = v
    return store[1:1 + 2 * v.size:2]


def _f32(v):
    return None if v is None else np.asarray(v, np.float32)


@pytest.mark.parametrize("c", batch_norm_cases(), ids=bn_case_id)
@pytest.mark.parametrize("channels_last", [False, True], ids=["planar", "interleaved"])
def test_golden_cases(c, channels_last):
    x, g, w, b = _f32(c["x"]), _f32(c["g"]), _strided(_f32(c["w"])), _strided(_f32(c["b"]))
    rm, rv = _strided(_f32(c["rm"])), _strided(_f32(c["rv"]))
    y, mean, inv, rm_out, rv_out = b200conv.batch_norm_forward(x, w, b, rm, rv, c["training"], c["momentum"], c["eps"],
                                                               channels_last=channels_last)
    stats = (mean, inv) if c["training"] else (rm, rv)
    dx, dw, db = b200conv.batch_norm_backward(g, x, w, *stats, c["training"], c["eps"], channels_last=channels_last)
    precise = c["tag"] == "precision"
    np.testing.assert_allclose(y, c["y"], rtol=4e-5 if precise else 3e-4, atol=2e-5 if precise else 3e-5)
    if c["training"]:
        np.testing.assert_allclose(mean, c["mean"], rtol=0 if precise else 3e-4, atol=1e-3 if precise else 3e-5)
        np.testing.assert_allclose(inv, c["inv"], rtol=4e-5, atol=2e-5)
    else:
        assert mean.size == 0 and inv.size == 0
    tol = dict(rtol=8e-5, atol=5e-5) if precise else dict(rtol=3e-4, atol=3e-5)
    np.testing.assert_allclose(dx, c["dx"], **tol)
    np.testing.assert_allclose(dw, c["dw"], **tol)
    np.testing.assert_allclose(db, c["db"], **tol)
    if c["rm_out"] is not None:
        np.testing.assert_allclose(rm_out, c["rm_out"], rtol=3e-4, atol=1e-3 if precise else 3e-5)
        np.testing.assert_allclose(rv_out, c["rv_out"], rtol=3e-4, atol=3e-5, equal_nan=True)
    if c["training"] and x.size // x.shape[1] == 2:   # equal and opposite, bit for bit
        pair = np.moveaxis(dx, 1, 0).reshape(x.shape[1], 2)
        np.testing.assert_array_equal(pair[:, 0], -pair[:, 1])


# rows arrangement (planes of 256 floats or more: aligned, unaligned, split into segments), columns
# arrangement (short planes, channels-last), channel counts off the vector width, a single image
SHAPES = [
    (4, 16, 32, 32), (3, 5, 33, 33), (1, 3, 96, 100), (2, 7, 20, 13), (8, 24, 14, 14), (16, 32, 7, 7),
    (5, 6, 7, 7), (64, 10), (300, 33), (2, 4, 3000), (1, 2, 5, 1000), (130, 8, 3, 3),
    # 64 channels or more of 32 to 256 KB each: one CTA per channel, one launch (planar layout)
    (32, 128, 7, 7), (16, 64, 28, 28), (12, 80, 33, 33), (64, 256, 14, 14), (3, 96, 5),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("channels_last", [False, True], ids=["planar", "interleaved"])
@pytest.mark.parametrize("training", [True, False], ids=["train", "eval"])
def test_against_the_fp64_oracle(shape, channels_last, training):
    rng = np.random.default_rng(sum(shape) + 7 * training)
    c = shape[1]
    x = (rng.standard_normal(shape) * 1.7 + 0.8).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    w, b = rng.standard_normal(c).astype(np.float32), rng.standard_normal(c).astype(np.float32)
    rm, rv = rng.standard_normal(c).astype(np.float32), (rng.random(c) + 0.4).astype(np.float32)
    y, mean, inv, rm_out, rv_out = b200conv.batch_norm_forward(x, w, b, rm, rv, training, 0.23, 1e-4, channels_last=channels_last)
    want = bn.forward(x, w, b, rm, rv, training, 0.23, 1e-4, dtype=np.float64)
    assert oracle.rel_l2(y, want[0]) <= GATE
    if training:
        np.testing.assert_allclose(mean, want[1], rtol=2e-6, atol=2e-6)
        np.testing.assert_allclose(inv, want[2], rtol=5e-6)
        np.testing.assert_allclose(rm_out, want[3], rtol=2e-6, atol=2e-6)
        np.testing.assert_allclose(rv_out, want[4], rtol=1e-5)
        stats = (mean, inv)
    else:
        np.testing.assert_array_equal(rm_out, rm)   # evaluation leaves the running statistics alone
        np.testing.assert_array_equal(rv_out, rv)
        stats = (rm, rv)
    dx, dw, db = b200conv.batch_norm_backward(g, x, w, *stats, training, 1e-4, channels_last=channels_last)
    wdx, wdw, wdb = bn.backward(g, x, w, *stats, training, 1e-4, dtype=np.float64)
    assert oracle.rel_l2(dx, wdx) <= 2 * GATE
    assert oracle.rel_l2(dw, wdw) <= 2 * GATE
    assert oracle.rel_l2(db, wdb) <= 2 * GATE
    channel_bytes = 4 * x.size // c
    one_launch = not channels_last and c >= 64 and 32 * 1024 <= channel_bytes <= 256 * 1024
    assert b200conv.last_kernel() == ("bn_backward_channel" if one_launch else b200conv.last_kernel())
    assert b200conv.last_kernel().startswith("bn_b")


@pytest.mark.parametrize("mask", [(True, False, False), (False, True, False), (False, False, True), (False, True, True),
                                  (False, False, False)])
@pytest.mark.parametrize("training", [True, False], ids=["train", "eval"])
def test_output_masks(mask, training):
    rng = np.random.default_rng(8)
    x, g = rng.standard_normal((2, 5, 7)).astype(np.float32), rng.standard_normal((2, 5, 7)).astype(np.float32)
    w, m, v = rng.standard_normal(5).astype(np.float32), rng.standard_normal(5).astype(np.float32), (rng.random(5) + .5).astype(np.float32)
    _, sm, si, _, _ = b200conv.batch_norm_forward(x, w, None, m, v, training, .1, 1e-5)
    stats = (sm, si) if training else (m, v)
    got = b200conv.batch_norm_backward(g, x, w, *stats, training, 1e-5, mask=mask)
    want = bn.backward(g, x, w, *stats, training, 1e-5, dtype=np.float64)
    for yes, a, e in zip(mask, got, want):
        if yes:
            np.testing.assert_allclose(a, e, rtol=3e-4, atol=3e-5)
        else:
            assert a is None


def test_absent_affine_and_running_statistics():
    rng = np.random.default_rng(11)
    x = rng.standard_normal((6, 4, 9, 9)).astype(np.float32)
    y, mean, inv, rm, rv = b200conv.batch_norm_forward(x, training=True, eps=1e-5)
    assert rm is None and rv is None
    want = bn.forward(x, training=True, eps=1e-5, dtype=np.float64)
    assert oracle.rel_l2(y, want[0]) <= GATE
    with pytest.raises(b200conv.B200Error, match="running statistics"):
        b200conv.batch_norm_forward(x, training=False)


def test_single_sample_gives_zero_output_and_nan_running_variance():
    x = np.ones((1, 3), np.float32)
    y, mean, inv, rm, rv = b200conv.batch_norm_forward(x, None, None, np.zeros(3, np.float32), np.ones(3, np.float32), True, .1, 1e-5)
    np.testing.assert_array_equal(y, np.zeros((1, 3), np.float32))
    assert np.isnan(rv).all()
    np.testing.assert_allclose(rm, 0.1 * np.ones(3), rtol=1e-6)


@pytest.mark.parametrize("channels_last", [False, True], ids=["planar", "interleaved"])
def test_constant_channel_and_zero_eps(channels_last):
    x = np.full((4, 3, 20, 20), 3.0, np.float32)
    y, mean, inv, _, _ = b200conv.batch_norm_forward(x, training=True, eps=0.0, channels_last=channels_last)
    np.testing.assert_array_equal(inv, np.zeros(3, np.float32))   # variance 0 and eps 0: inverse defined as 0
    np.testing.assert_array_equal(y, np.zeros_like(x))
    np.testing.assert_array_equal(mean, np.full(3, 3.0, np.float32))


@pytest.mark.parametrize("shape", [(8, 4, 64, 64), (4096, 8)], ids=["rows", "columns"])
def test_statistics_survive_a_large_offset_and_an_outlier_at_the_origin(shape):
    # the channel origin (first element) is far from the rest: a shift by the origin alone would
    # lose the variance to cancellation; the reference's second, centred pass does not, nor may this
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(shape) * 0.1 + 10000.0).astype(np.float32)
    x[0] = 0.0
    y, mean, inv, _, _ = b200conv.batch_norm_forward(x, training=True, eps=1e-5)
    want = bn.forward(x, training=True, eps=1e-5, dtype=np.float64)
    # with the origin at 0 the mean is held relative to 0: two units in the last place of 1e4
    np.testing.assert_allclose(mean, want[1], rtol=0, atol=2e-3)
    np.testing.assert_allclose(inv, want[2], rtol=1e-3)
    x = (rng.standard_normal(shape) * 0.1 + 10000.0).astype(np.float32)   # offset only
    y, mean, inv, _, _ = b200conv.batch_norm_forward(x, training=True, eps=1e-5)
    want = bn.forward(x, training=True, eps=1e-5, dtype=np.float64)
    np.testing.assert_allclose(inv, want[2], rtol=3e-5, atol=1e-5)
    np.testing.assert_allclose(y, want[0], rtol=3e-4, atol=0.008)


@pytest.mark.parametrize("channels_last", [False, True], ids=["planar", "interleaved"])
def test_full_size_layer_properties(channels_last):
    # 64 x 64 x 56 x 56 (the first sweep layer's activation): normalised output has zero mean and unit
    # variance per channel, dx is orthogonal to 1 and to the normalised input, and the whole tensor
    # matches the FP64 oracle
    rng = np.random.default_rng(21)
    shape = (64, 64, 56, 56)
    x = (rng.standard_normal(shape, dtype=np.float32) * 2.0 + 1.5)
    g = rng.standard_normal(shape, dtype=np.float32)
    y, mean, inv, _, _ = b200conv.batch_norm_forward(x, training=True, eps=1e-5, channels_last=channels_last)
    rows = np.moveaxis(y, 1, 0).reshape(64, -1).astype(np.float64)
    assert np.abs(rows.mean(axis=1)).max() < 1e-5
    np.testing.assert_allclose(rows.var(axis=1), 1.0, rtol=1e-4)
    dx, dw, db = b200conv.batch_norm_backward(g, x, None, mean, inv, True, 1e-5, channels_last=channels_last)
    drows = np.moveaxis(dx, 1, 0).reshape(64, -1).astype(np.float64)
    scale = np.abs(drows).sum(axis=1)
    assert (np.abs(drows.sum(axis=1)) / scale).max() < 1e-5
    assert (np.abs((drows * rows).sum(axis=1)) / scale).max() < 1e-5
    want = bn.forward(x, training=True, eps=1e-5, dtype=np.float64)
    assert oracle.rel_l2(y, want[0]) <= GATE
    wdx, wdw, wdb = bn.backward(g, x, None, want[1], want[2], True, 1e-5, dtype=np.float64)
    assert oracle.rel_l2(dx, wdx) <= 2 * GATE
    assert oracle.rel_l2(dw, wdw) <= 1e-4 and oracle.rel_l2(db, wdb) <= 1e-4


def test_invalid_arguments():
    L = b200conv.lib()
    b200conv.init()
    assert L.b200_batch_norm_workspace(0, 3, 4, 0) == 0
    assert L.b200_batch_norm_workspace(2, 3, 4, 7) == 0
    with pytest.raises(ValueError, match="shape mismatch"):
        b200conv.batch_norm_backward(np.zeros((2, 3, 4), np.float32), np.zeros((2, 3, 5), np.float32), None,
                                     np.zeros(3, np.float32), np.ones(3, np.float32))


@pytest.mark.parametrize("shape", [(4, 16, 32, 32), (3, 5, 33, 33), (16, 32, 7, 7), (300, 33), (8, 24, 14, 14), (48, 64, 14, 14), (6, 72, 9, 7)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("channels_last", [False, True], ids=["planar", "interleaved"])
@pytest.mark.parametrize("training", [True, False], ids=["train", "eval"])
@pytest.mark.parametrize("ops", ["relu", "residual", "residual_relu"])
def test_fused_residual_and_relu(shape, channels_last, training, ops):
    rng = np.random.default_rng(sum(shape) + len(ops))
    c = shape[1]
    x = (rng.standard_normal(shape) * 1.3 - 0.2).astype(np.float32)
    res = rng.standard_normal(shape).astype(np.float32) if "residual" in ops else None
    w, b = rng.standard_normal(c).astype(np.float32), rng.standard_normal(c).astype(np.float32)
    rm, rv = rng.standard_normal(c).astype(np.float32), (rng.random(c) + 0.4).astype(np.float32)
    relu = "relu" in ops
    y, mean, inv, rm_out, rv_out = b200conv.batch_norm_forward(x, w, b, rm, rv, training, 0.1, 1e-5, channels_last=channels_last,
                                                               residual=res, relu=relu)
    assert "fused" in b200conv.last_kernel()
    want = bn.forward(x, w, b, rm, rv, training, 0.1, 1e-5, dtype=np.float64)
    ref = want[0] + (res if res is not None else 0.0)
    if relu:
        ref = np.maximum(ref, 0.0)
        assert (y >= 0).all()
    assert oracle.rel_l2(y, ref) <= GATE
    # the statistics are those of the plain call
    plain = b200conv.batch_norm_forward(x, w, b, rm, rv, training, 0.1, 1e-5, channels_last=channels_last)
    for a, e in zip((mean, inv, rm_out, rv_out), plain[1:]):
        np.testing.assert_array_equal(a, e)
