"""BASELINE configurations 3, 4 and 5 through the C-ABI on the GPU.

Reduced batches are compared with the PyTorch-CPU FP64 oracle; the full sizes are checked through
size-independent properties of convolution (the adjoint identities
<conv(x,w), dy> = <x, dInput(dy,w)> = <w, dWeight(x,dy)>, and linearity in x), evaluated in FP64 on
the host from the kernels' FP32 outputs."""
import numpy as np
import pytest

import b200conv
import dp
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-4


def _rng(seed):
    return np.random.default_rng(seed)


def _check(x, w, b, go, want=None, **args):
    y = b200conv.conv2d_forward(x, w, b, **args)
    dx, dw, db = b200conv.conv2d_backward(go, x, w, **args)
    assert b200conv.device_status() == 0
    if want is None:
        want = oracle.torch_conv_all(np.ascontiguousarray(x), np.ascontiguousarray(w), b, np.ascontiguousarray(go),
                                     args.get("stride", (1, 1)), args.get("padding", (0, 0)),
                                     args.get("dilation", (1, 1)), args.get("groups", 1))
    errs = [oracle.rel_l2(a, e) for a, e in zip((y, dx, dw, db), want)]
    assert max(errs) <= GATE, errs
    return y, dx, dw, db


# ---- config 3: 3x3 stride-1 pad-1, weights N(0, 0.02), incl. odd 33x33 maps ----------------------
@pytest.mark.parametrize("c,hw", [(64, 16), (64, 33), (128, 32), (256, 16), (512, 16), (128, 33)])
def test_config3_same_size_3x3_layers(c, hw):
    r = _rng(2000 + c + hw)
    n = 2
    x = r.standard_normal((n, c, hw, hw), dtype=np.float32)
    w = (r.standard_normal((c, c, 3, 3), dtype=np.float32) * 0.02).astype(np.float32)
    b = (r.standard_normal(c, dtype=np.float32) * 0.02).astype(np.float32)
    go = r.standard_normal((n, c, hw, hw), dtype=np.float32)
    _check(x, w, b, go, padding=(1, 1))


# ---- config 4: U-Net style mix on sliced/offset views ------------------------------------------------
UNET = [
    # (cin, cout, hw, kernel, kwargs)
    (128, 128, 32, (3, 3), dict(padding=(1, 1))),
    (256, 256, 16, (3, 3), dict(padding=(1, 1), groups=32)),
    (512, 512, 8, (3, 3), dict(padding=(1, 1), groups=32)),
    (128, 128, 32, (3, 3), dict(padding=(2, 2), dilation=(2, 2))),
    (128, 256, 32, (3, 3), dict(stride=(2, 2), padding=(1, 1))),
    (128, 256, 32, (1, 1), dict()),
]


@pytest.mark.parametrize("spec", UNET, ids=lambda s: f"{s[0]}-{s[1]}-{s[2]}-k{s[3][0]}-" + "-".join(f"{k}{v}" for k, v in s[4].items()))
@pytest.mark.parametrize("channels_last", [False, True], ids=["view", "view-nhwc"])
def test_config4_unet_mix_on_strided_views(spec, channels_last):
    cin, cout, hw, kernel, kw = spec
    r = _rng(3000 + cin + cout + hw)
    n = 2
    base = r.standard_normal((n, cin + 8, hw + 2, hw + 2), dtype=np.float32)
    if channels_last:
        base = np.ascontiguousarray(base.transpose(0, 2, 3, 1)).transpose(0, 3, 1, 2)
    x = base[:, 4:4 + cin, 1:1 + hw, 1:1 + hw]           # offset + non-dense strides, consumed in place
    groups = kw.get("groups", 1)
    fan_in = (cin // groups) * kernel[0] * kernel[1]
    w = ((r.random((cout, cin // groups, *kernel), dtype=np.float32) * 2 - 1) / np.sqrt(fan_in)).astype(np.float32)
    b = ((r.random(cout, dtype=np.float32) * 2 - 1) / np.sqrt(fan_in)).astype(np.float32)
    g = oracle.geometry(x.shape, cout, kernel, **kw)
    go = r.standard_normal(g.y_shape, dtype=np.float32)
    _check(x, w, b, go, **kw)


# ---- config 5: batch sharded over ranks, dW/dB summed ----------------------------------------------------
def test_config5_sharded_gradients_equal_the_full_batch(world=4):
    c, hw, global_batch = 256, 14, 16
    gw = np.random.default_rng(4999)
    w = ((gw.random((c, c, 3, 3), dtype=np.float32) * 2 - 1) / np.sqrt(c * 9)).astype(np.float32)
    b = ((gw.random(c, dtype=np.float32) * 2 - 1) / np.sqrt(c * 9)).astype(np.float32)
    x_full = dp.seeded_samples((c, hw, hw), 5000, 0, global_batch).numpy()
    go_full = dp.seeded_samples((c, hw, hw), 7000, 0, global_batch).numpy()
    want = oracle.torch_conv_all(x_full, w, b, go_full, (1, 1), (1, 1), (1, 1), 1)
    dw_sum = np.zeros_like(w, dtype=np.float64)
    db_sum = np.zeros(c, np.float64)
    for rank in range(world):
        lo, hi = dp.shard_range(global_batch, rank, world)
        x = dp.seeded_samples((c, hw, hw), 5000, lo, hi).numpy()     # each rank regenerates its own slice
        go = dp.seeded_samples((c, hw, hw), 7000, lo, hi).numpy()
        y = b200conv.conv2d_forward(x, w, b, padding=(1, 1))
        dx, dw, db = b200conv.conv2d_backward(go, x, w, padding=(1, 1))
        assert oracle.rel_l2(y, want[0][lo:hi]) <= GATE        # forward and dInput are rank-local
        assert oracle.rel_l2(dx, want[1][lo:hi]) <= GATE
        dw_sum += dw
        db_sum += db
    assert oracle.rel_l2(dw_sum, want[2]) <= GATE
    assert oracle.rel_l2(db_sum, want[3]) <= GATE


# ---- full-size properties -----------------------------------------------------------------------------------
def _dot(a, b):
    return float(np.dot(a.ravel().astype(np.float64), b.ravel().astype(np.float64)))


@pytest.mark.parametrize("shape", [
    (64, 64, 64, 56, (3, 3), dict(padding=(1, 1))),                    # sweep layer, full batch
    (32, 256, 256, 32, (3, 3), dict(padding=(1, 1))),                  # config 3, full batch
    (64, 128, 128, 56, (3, 3), dict(stride=(2, 2), padding=(1, 1))),   # stride-2 sweep layer
    (64, 256, 64, 56, (1, 1), dict()),                                 # 1x1 sweep layer
    (16, 256, 256, 32, (3, 3), dict(padding=(1, 1), groups=32)),       # config 4 grouped
], ids=lambda s: f"n{s[0]}-{s[1]}to{s[2]}-{s[3]}sq-k{s[4][0]}")
def test_adjoint_identities_and_linearity_at_full_size(shape):
    n, cin, cout, hw, kernel, kw = shape
    r = _rng(n + cin + cout + hw)
    groups = kw.get("groups", 1)
    x = r.standard_normal((n, cin, hw, hw), dtype=np.float32)
    x2 = r.standard_normal((n, cin, hw, hw), dtype=np.float32)
    w = (r.standard_normal((cout, cin // groups, *kernel), dtype=np.float32) / np.sqrt(cin // groups * kernel[0] * kernel[1])).astype(np.float32)
    g = oracle.geometry(x.shape, cout, kernel, **kw)
    go = r.standard_normal(g.y_shape, dtype=np.float32)
    y = b200conv.conv2d_forward(x, w, None, **kw)
    dx, dw, db = b200conv.conv2d_backward(go, x, w, **kw)
    assert b200conv.device_status() == 0
    lhs = _dot(y, go)
    scale = np.linalg.norm(y.astype(np.float64)) * np.linalg.norm(go.astype(np.float64))
    assert abs(lhs - _dot(x, dx)) <= GATE * scale
    assert abs(lhs - _dot(w, dw)) <= GATE * scale
    np.testing.assert_allclose(db, go.astype(np.float64).sum(axis=(0, 2, 3)), rtol=1e-4, atol=1e-2)
    y2 = b200conv.conv2d_forward(x2, w, None, **kw)
    y12 = b200conv.conv2d_forward((0.5 * x - 2.0 * x2).astype(np.float32), w, None, **kw)
    assert oracle.rel_l2(y12, 0.5 * y.astype(np.float64) - 2.0 * y2.astype(np.float64)) <= GATE
