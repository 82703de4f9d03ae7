"""Seeded random geometries through the C ABI with the automatic candidate choice, all four phases against PyTorch CPU
FP64 on the same inputs.  The hand-picked cases elsewhere pin each kernel on shapes chosen for it; this sweep draws the
shapes (channel counts on and off the 16 / 32 / 64 / 128 boundaries, ragged images, strides 1-3, dilation, groups,
kernels 1 to 5 wide, both layouts, sliced views) so that whatever the heuristic routes them to -- direct, tiled,
grouped-small, strip, transposed strip, gather, the 16-producer instances -- is compared with the oracle."""
import numpy as np
import pytest

import b200conv
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-4     # the contract's gate: the candidate is whatever AUTO picks, CUDA-core FP32 or split-precision tcgen05

CHANNELS = (8, 16, 24, 32, 48, 64, 72, 96, 128, 144, 192, 256)


def _draw(rng):
    while True:
        groups = int(rng.choice((1, 1, 1, 2, 4, 8)))
        cin, cout = int(rng.choice(CHANNELS)), int(rng.choice(CHANNELS))
        if cin % groups or cout % groups:
            continue
        kh, kw = int(rng.choice((1, 2, 3, 3, 3, 5))), int(rng.choice((1, 2, 3, 3, 3, 5)))
        sh, sw = int(rng.choice((1, 1, 1, 2, 3))), int(rng.choice((1, 1, 1, 2, 3)))
        dh, dw = int(rng.choice((1, 1, 2))), int(rng.choice((1, 1, 2)))
        ph, pw = int(rng.integers(0, dh * (kh - 1) // 2 + 2)), int(rng.integers(0, dw * (kw - 1) // 2 + 2))
        h, w = int(rng.integers(4, 41)), int(rng.integers(4, 41))
        if h + 2 * ph < dh * (kh - 1) + 1 or w + 2 * pw < dw * (kw - 1) + 1:
            continue
        n = int(rng.integers(1, 5))
        if n * cin * h * w > 1 << 21:            # keep the FP64 reference quick
            continue
        layout = str(rng.choice(("nchw", "nhwc", "sliced")))
        return dict(xshape=(n, cin, h, w), cout=cout, kernel=(kh, kw), stride=(sh, sw), padding=(ph, pw), dilation=(dh, dw),
                    groups=groups, layout=layout)


def _cases(count, seed):
    rng = np.random.default_rng(seed)
    return [_draw(rng) for _ in range(count)]


def _as_layout(a, layout):
    if layout == "nhwc":
        return np.ascontiguousarray(a.transpose(0, 2, 3, 1)).transpose(0, 3, 1, 2)
    if layout == "sliced":   # an offset view with non-dense strides inside a larger parent
        n, c, h, w = a.shape
        parent = np.zeros((n, c + 3, h + 2, w + 5), np.float32)
        view = parent[:, 2:2 + c, 1:1 + h, 3:3 + w]
        view[...] = a
        return view
    return a


@pytest.mark.parametrize("case", _cases(160, 20261), ids=lambda c: "{}-co{}-k{}-s{}-p{}-d{}-g{}-{}".format(
    "x".join(map(str, c["xshape"])), c["cout"], "x".join(map(str, c["kernel"])), "x".join(map(str, c["stride"])),
    "x".join(map(str, c["padding"])), "x".join(map(str, c["dilation"])), c["groups"], c["layout"]))
def test_random_geometry_all_phases(case):
    args = dict(stride=case["stride"], padding=case["padding"], dilation=case["dilation"], groups=case["groups"])
    g = oracle.geometry(case["xshape"], case["cout"], case["kernel"], **args)
    rng = np.random.default_rng(sum(case["xshape"]) + 17 * case["cout"])
    x = rng.standard_normal(g.x_shape, dtype=np.float32)
    w = (rng.standard_normal(g.w_shape, dtype=np.float32) / np.sqrt(np.prod(g.w_shape[1:]))).astype(np.float32)
    b = rng.standard_normal(case["cout"], dtype=np.float32)
    go = rng.standard_normal(g.y_shape, dtype=np.float32)
    want = oracle.torch_conv_all(x, w, b, go, args["stride"], args["padding"], args["dilation"], args["groups"])
    xv, gov = _as_layout(x, case["layout"]), _as_layout(go, case["layout"])
    y = b200conv.conv2d_forward(xv, w, b, **args)
    fwd_kernel = b200conv.last_kernel()
    dx, dw, db = b200conv.conv2d_backward(gov, xv, w, **args)
    assert b200conv.device_status() == 0
    errs = [oracle.rel_l2(a, e) for a, e in zip((y, dx, dw, db), want)]
    assert max(errs) <= GATE, (fwd_kernel, errs)


def _draw_wide(rng):
    """Layers of tensor-core size: 64 to 512 channels, images up to 48x48, batches up to 8."""
    while True:
        groups = int(rng.choice((1, 1, 1, 2)))
        cin, cout = int(rng.choice((64, 80, 128, 160, 256, 320, 512))), int(rng.choice((64, 80, 128, 160, 256, 320, 512)))
        k = int(rng.choice((1, 2, 3, 3, 3)))
        s = int(rng.choice((1, 1, 2)))
        d = int(rng.choice((1, 1, 2)))
        p = int(rng.integers(0, d * (k - 1) // 2 + 2))
        h, w = int(rng.integers(7, 49)), int(rng.integers(7, 49))
        n = int(rng.integers(2, 9))
        if h + 2 * p < d * (k - 1) + 1 or w + 2 * p < d * (k - 1) + 1 or n * max(cin, cout) * h * w > 3 << 21:
            continue
        return dict(xshape=(n, cin, h, w), cout=cout, kernel=(k, k), stride=(s, s), padding=(p, p), dilation=(d, d), groups=groups,
                    layout=str(rng.choice(("nchw", "nhwc"))))


@pytest.mark.parametrize("case", [_draw_wide(r) for r in [np.random.default_rng(77)] for _ in range(48)],
                         ids=lambda c: "{}-co{}-k{}-s{}-p{}-d{}-g{}-{}".format("x".join(map(str, c["xshape"])), c["cout"], c["kernel"][0],
                                                                              c["stride"][0], c["padding"][0], c["dilation"][0],
                                                                              c["groups"], c["layout"]))
def test_random_tensor_core_layers(case):
    """The tcgen05 candidates forced on random wide layers (strip, transposed strip, their 16-producer instances, the
    chunked dWeight): 2.5e-5, the split-precision kernels' own bound, not the contract's 1e-4."""
    args = dict(stride=case["stride"], padding=case["padding"], dilation=case["dilation"], groups=case["groups"])
    g = oracle.geometry(case["xshape"], case["cout"], case["kernel"], **args)
    rng = np.random.default_rng(sum(case["xshape"]) + 31 * case["cout"])
    x = rng.standard_normal(g.x_shape, dtype=np.float32)
    w = (rng.standard_normal(g.w_shape, dtype=np.float32) / np.sqrt(np.prod(g.w_shape[1:]))).astype(np.float32)
    b = rng.standard_normal(case["cout"], dtype=np.float32)
    go = rng.standard_normal(g.y_shape, dtype=np.float32)
    want = oracle.torch_conv_all(x, w, b, go, args["stride"], args["padding"], args["dilation"], args["groups"])
    xv, gov = _as_layout(x, case["layout"]), _as_layout(go, case["layout"])
    y = b200conv.conv2d_forward(xv, w, b, algo="tc", budget=1 << 30, **args)
    assert b200conv.last_kernel().startswith("tc_")
    dx, dw, db = b200conv.conv2d_backward(gov, xv, w, algo="tc", budget=1 << 30, **args)
    assert b200conv.device_status() == 0
    errs = [oracle.rel_l2(a, e) for a, e in zip((y, dx, dw, db), want)]
    assert max(errs) <= 2.5e-5, errs
