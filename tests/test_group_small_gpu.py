"""Grouped 3x3 convolutions with 4 or 8 channels per group (the groups=32 layers of a U-Net block): the kernels whose
tile follows the group, against the PyTorch-CPU FP64 oracle.  FP32 FMA arithmetic: held to 5e-6 (contract: 1e-4)."""
import numpy as np
import pytest

import b200conv
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 5e-6


def _nhwc(a):
    return np.ascontiguousarray(a.transpose(0, 2, 3, 1)).transpose(0, 3, 1, 2)


@pytest.mark.parametrize("n,c,groups,h,w", [
    (2, 128, 32, 64, 64),     # 4 per group, whole tiles
    (3, 64, 8, 19, 70),       # 8 per group, ragged rows and columns (two column tiles)
    (1, 16, 4, 5, 3),         # smaller than a tile
    (2, 256, 32, 32, 32),     # 8 per group
    (5, 8, 2, 33, 129),       # 4 per group, three column tiles
], ids=lambda v: str(v))
@pytest.mark.parametrize("layout", ["nchw", "nhwc", "view"])
def test_small_group_kernels_match_the_oracle(n, c, groups, h, w, layout):
    rng = np.random.default_rng(n + c + h + w)
    cpg = c // groups
    if layout == "view":
        base = rng.standard_normal((n, c + 8, h + 2, w + 2), dtype=np.float32)
        x = base[:, 4:4 + c, 1:1 + h, 1:1 + w]
    else:
        x = rng.standard_normal((n, c, h, w), dtype=np.float32)
    go = rng.standard_normal((n, c, h, w), dtype=np.float32)
    if layout == "nhwc":
        x, go = _nhwc(x), _nhwc(go)
    wt = (rng.standard_normal((c, cpg, 3, 3), dtype=np.float32) / np.sqrt(cpg * 9)).astype(np.float32)
    b = rng.standard_normal(c, dtype=np.float32)
    kw = dict(padding=(1, 1), groups=groups)
    want = oracle.torch_conv_all(np.ascontiguousarray(x), wt, b, np.ascontiguousarray(go), (1, 1), (1, 1), (1, 1), groups)
    y = b200conv.conv2d_forward(x, wt, b, **kw)
    assert b200conv.last_kernel() == "group_small_forward"
    dx, dw, db = b200conv.conv2d_backward(go, x, wt, **kw)
    errs = [oracle.rel_l2(a, e) for a, e in zip((y, dx, dw, db), want)]
    assert max(errs) <= GATE, errs
    # the same result from run to run (ordered sums, no atomics)
    dw2 = b200conv.conv2d_backward(go, x, wt, mask=(False, True, False), **kw)[1]
    np.testing.assert_array_equal(dw, dw2)
    # without scratch the weight gradient falls back to the implicit-GEMM kernel and still agrees
    dw3 = b200conv.conv2d_backward(go, x, wt, mask=(False, True, False), budget=0, **kw)[1]
    assert oracle.rel_l2(dw3, want[2]) <= GATE


def test_other_grouped_shapes_keep_the_general_kernels():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 16, 9, 9), dtype=np.float32)
    for cout, kernel, kw in ((32, (3, 3), dict(padding=(1, 1), groups=4)),           # 4 in, 8 out per group
                             (16, (3, 3), dict(padding=(1, 1), groups=4, stride=(2, 2))),
                             (16, (5, 5), dict(padding=(2, 2), groups=4))):
        w = rng.standard_normal((cout, 4, *kernel), dtype=np.float32)
        y = b200conv.conv2d_forward(x, w, None, **kw)
        assert b200conv.last_kernel() != "group_small_forward"
        want = oracle.torch_conv_all(x, w, None, np.zeros_like(y), kw.get("stride", (1, 1)), kw["padding"], (1, 1), 4)[0]
        assert oracle.rel_l2(y, want) <= GATE
