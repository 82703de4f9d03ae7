"""Pins the CPU oracle: golden vectors (PyTorch CPU FP64 on the reference's seeded
cases) and the closed-form known-answer cases the reference's tests hold."""
import numpy as np
import pytest

from golden_cases import case_id, conv_cases, gemm_cases
from oracle import oracle

CASES = conv_cases()


def _geom(c):
    return oracle.geometry(c["xshape"], c["cout"], c["kernel"], c["stride"], c["padding"], c["dilation"],
                           c["groups"])


def _close(actual, expected, rtol, atol):
    np.testing.assert_allclose(actual, expected, rtol=rtol, atol=atol)


@pytest.mark.parametrize("c", CASES, ids=case_id)
def test_direct_order_matches_golden(c):
    # tolerances of tests/test_conv_dispatch.py:67,70 (scaled by input magnitude for unit-scale cases)
    g = _geom(c)
    s = 1.0 if c["tag"] == "dispatch" else 10.0
    _close(oracle.forward(g, c["x"], c["w"], c["b"]), c["y"], 4e-4, 3e-5 * s)
    _close(oracle.dinput(g, c["go"], c["w"]), c["dx"], 5e-4, 5e-5 * s)
    _close(oracle.dweight(g, c["x"], c["go"]), c["dw"], 5e-4, 5e-5 * s)
    _close(oracle.dbias(g, c["go"]), c["db"], 5e-4, 5e-5 * s)


@pytest.mark.parametrize("c", CASES, ids=case_id)
def test_f64_accumulation_matches_golden_tightly(c):
    g = _geom(c)
    for got, want in ((oracle.forward(g, c["x"], c["w"], c["b"], f64=True), c["y"]),
                      (oracle.dinput(g, c["go"], c["w"], f64=True), c["dx"]),
                      (oracle.dweight(g, c["x"], c["go"], f64=True), c["dw"]),
                      (oracle.dbias(g, c["go"], f64=True), c["db"])):
        assert oracle.rel_l2(got, want) < 2e-7


@pytest.mark.parametrize("c", CASES, ids=case_id)
def test_tiled_and_reduce_orders_match_golden(c):
    g = _geom(c)
    s = 1.0 if c["tag"] == "dispatch" else 10.0
    _close(oracle.forward(g, c["x"], c["w"], c["b"], order="tiled"), c["y"], 4e-4, 3e-5 * s)
    _close(oracle.dinput(g, c["go"], c["w"], order="tiled"), c["dx"], 5e-4, 5e-5 * s)
    _close(oracle.dweight(g, c["x"], c["go"], order="reduce"), c["dw"], 5e-4, 5e-5 * s)
    _close(oracle.dbias(g, c["go"], order="reduce"), c["db"], 5e-4, 5e-5 * s)
    for span in (16, 256):
        _close(oracle.dweight(g, c["x"], c["go"], order="split", span=span), c["dw"], 5e-4, 5e-5 * s)


@pytest.mark.parametrize("c", [c for c in CASES if c["kernel"] == (3, 3) and c["stride"] == (1, 1)
                               and c["dilation"] == (1, 1)], ids=case_id)
def test_winograd_f2_matches_golden(c):
    g = _geom(c)
    s = 1.0 if c["tag"] == "dispatch" else 10.0
    _close(oracle.forward(g, c["x"], c["w"], c["b"], order="winograd_f2"), c["y"], 4e-4, 3e-5 * s)


@pytest.mark.parametrize("c", [c for c in CASES if c["groups"] == c["xshape"][1] and c["groups"] > 1], ids=case_id)
def test_depthwise_matches_golden(c):
    g = _geom(c)
    _close(oracle.forward(g, c["x"], c["w"], c["b"], order="depthwise"), c["y"], 4e-4, 3e-4)


def test_known_answer_affine_forward_and_constant_dinput():
    # tests/test_conv_dispatch.py:315-333: x = arange % 97 / 97, 1x1 weight 2, bias 1 -> 2x+1 exactly;
    # dX with a constant 0.25 gradient -> exactly 0.5 (rtol = atol = 0).
    n = 70000
    x = ((np.arange(n) % 97) / 97.0).astype(np.float32).reshape(1, 1, 1, n)
    w = np.full((1, 1, 1, 1), 2.0, np.float32)
    b = np.ones(1, np.float32)
    g = oracle.geometry(x.shape, 1, (1, 1))
    for order in ("direct", "tiled"):
        np.testing.assert_array_equal(oracle.forward(g, x, w, b, order=order), 2 * x + 1)
    go = np.full(g.y_shape, 0.25, np.float32)
    for order in ("direct", "tiled"):
        np.testing.assert_array_equal(oracle.dinput(g, go, w, order=order), np.full(x.shape, 0.5, np.float32))


def test_known_answer_mm_2x2():
    # tests/test_mm.py:29-36
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[5, 6], [7, 8]], np.float32)
    np.testing.assert_array_equal(oracle.gemm(a, b), np.array([[19, 22], [43, 50]], np.float32))


def test_gemm_matches_golden_with_transposed_operand():
    for case in gemm_cases():
        for (beta, alpha), want in zip(case["scalars"], case["outs"]):
            got = oracle.gemm(case["a"], case["bt"].T, case["bias"], alpha=alpha, beta=beta)
            np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-4)
            got64 = oracle.gemm(case["a"], case["bt"].T, case["bias"], alpha=alpha, beta=beta, f64=True)
            assert oracle.rel_l2(got64, want) < 2e-7


def test_beta_zero_does_not_read_bias():
    # matmul_strided_bias.comp:66 / mm.cpp:914-915: beta == 0 must not propagate NaN from the bias
    a = np.ones((3, 4), np.float32)
    b = np.ones((4, 5), np.float32)
    bias = np.full(5, np.nan, np.float32)
    assert np.isfinite(oracle.gemm(a, b, bias, alpha=1.0, beta=0.0)).all()


def test_geometry_rejections():
    # tests/test_conv_universality.py:96-101: a 3x3 filter over a 2x2 map with stride 2 must raise
    with pytest.raises(ValueError, match="effective kernel"):
        oracle.geometry((1, 2, 2, 2), 3, (3, 3), stride=(2, 2))
    with pytest.raises(ValueError, match="int32 coordinates"):
        oracle.geometry((1, 1, 4, 4), 1, (1, 1), stride=(2 ** 31, 1))
    with pytest.raises(ValueError, match="invalid shapes"):
        oracle.geometry((1, 6, 4, 4), 4, (1, 1), groups=4)


def test_weight_split_plan():
    # csrc/ops/convolution.cpp:204-238
    g = oracle.geometry((8, 64, 56, 56), 64, (3, 3), padding=(1, 1))
    span, count, nbytes = oracle.weight_split_plan(g)
    assert (span, count) == (256, 98) and nbytes == 98 * 64 * 64 * 9 * 4
    g = oracle.geometry((1, 9, 1, 256), 17, (1, 1))
    assert oracle.weight_split_plan(g) == (256, 1, 0)
    g = oracle.geometry((1, 9, 1, 257), 17, (1, 1))
    assert oracle.weight_split_plan(g)[:2] == (256, 2)
    # budget-limited: fewer, longer, tile-aligned spans
    g = oracle.geometry((64, 256, 56, 56), 256, (3, 3), padding=(1, 1))
    span, count, nbytes = oracle.weight_split_plan(g)
    assert nbytes <= 64 << 20 and span % 16 == 0 and count == -(-(64 * 56 * 56) // span)
    assert oracle.weight_split_plan(g, budget=0)[1] == 0


def test_pack_strided_views():
    base = np.arange(3 * 6 * 13 * 15, dtype=np.float32).reshape(3, 6, 13, 15)
    for view in (base.transpose(0, 1, 3, 2), base[:, :, 1::2, ::2], base[1:],
                 np.broadcast_to(base[:1], (3, 6, 13, 15))):
        off = (view.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // 4
        got = oracle.pack(base, off, view.shape, [s // 4 for s in view.strides])
        np.testing.assert_array_equal(got, np.ascontiguousarray(view))
