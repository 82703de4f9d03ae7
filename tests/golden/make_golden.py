"""Generate the committed golden vectors for the Conv2D / GEMM hot path.

Run here (CPU only):  python tests/golden/make_golden.py

The reference holds no stored numeric fixtures for this path: every one of its
convolution tests draws seeded CPU tensors and compares the device result with
PyTorch's CPU convolution, in FP32 (tests/test_convolution.py:21-40,
tests/test_conv_universality.py:25-44) or promoted to FP64
(tests/test_conv_dispatch.py:50-70).  This script reproduces those draws (same
seeds, same order of generator calls, same scale factors, same geometries) and
stores inputs together with the PyTorch-CPU FP64 results rounded to FP32, so
that the oracle and the CUDA path can be checked against the reference's own
ground truth on a machine where PyTorch's generator is not trusted to be
bit-stable.  Closed-form known-answer cases (tests/test_conv_dispatch.py:315-333,
tests/test_mm.py:29-36) are stated in tests/test_oracle.py instead.

Output: tests/golden/conv_cases.npz, tests/golden/gemm_cases.npz (about 1 MB together).
"""
import os

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))

# (xshape, cout, kernel, stride, padding, dilation, groups): the geometry rows of
# tests/test_conv_dispatch.py:20-47 (ragged-tile boundaries, large filters,
# grouped/strided/dilated, depthwise multiplier, split boundaries 255/256/257).
DISPATCH_CASES = [
    ((1, 7, 1, 15), 7, (1, 1), (1, 1), (0, 0), (1, 1), 1),
    ((1, 9, 1, 17), 9, (1, 1), (1, 1), (0, 0), (1, 1), 1),
    ((1, 15, 1, 31), 15, (1, 1), (1, 1), (0, 0), (1, 1), 1),
    ((1, 17, 1, 33), 17, (1, 1), (1, 1), (0, 0), (1, 1), 1),
    ((1, 31, 1, 63), 31, (1, 1), (1, 1), (0, 0), (1, 1), 1),
    ((1, 33, 1, 65), 33, (1, 1), (1, 1), (0, 0), (1, 1), 1),
    *[((1, 9, k + 3, k + 5), 17, (k, k), (1, 1), (0, 0), (1, 1), 1) for k in (9, 10, 11, 12)],
    ((2, 18, 19, 23), 34, (3, 5), (2, 1), (2, 3), (2, 1), 2),
    ((1, 5, 11, 13), 15, (3, 5), (1, 2), (1, 4), (1, 2), 5),
    ((2, 6, 15, 19), 9, (3, 5), (1, 1), (3, 4), (2, 3), 3),
    ((1, 5, 11, 13), 15, (3, 5), (1, 1), (2, 4), (2, 2), 5),
    ((1, 9, 17, 23), 17, (3, 5), (2, 3), (3, 2), (2, 1), 1),
    *[((1, 9, 1, pos), 17, (1, 1), (1, 1), (0, 0), (1, 1), 1) for pos in (255, 256, 257)],
]

# tests/test_convolution.py:8-13 (seed 72, unit-scale randn, square kernel ints)
BASIC_CASES = [
    ((2, 3, 9, 11), 4, 3, 1, 1, 1, 1, True),
    ((1, 2, 11, 12), 3, 3, 2, 1, 1, 1, False),
    ((2, 4, 8, 7), 6, 3, 1, 2, 2, 2, True),
    ((1, 8, 8, 8), 8, 1, 1, 0, 1, 8, True),
]

# tests/test_conv_universality.py:14-21 (seed = sum(xshape)+cout+sum(kernel))
UNIVERSAL_CASES = [
    ((2, 9, 17, 19), 19, (1, 1), (1, 1), (0, 0), (1, 1), 1),
    ((2, 9, 17, 19), 19, (5, 5), (2, 1), (3, 2), (2, 1), 1),
    ((1, 2, 14, 15), 3, (3, 5), (2, 1), (1, 2), (1, 2), 1),
    ((1, 1, 13, 14), 2, (7, 7), (1, 1), (3, 3), (1, 1), 1),
    ((1, 4, 11, 12), 12, (3, 3), (1, 1), (1, 1), (1, 1), 4),
    ((2, 6, 9, 10), 9, (5, 1), (1, 2), (2, 0), (1, 1), 3),
]

# Winograd-gated shapes of tests/test_conv_dispatch.py:440-510: odd-sized map (scaled to 19x21),
# grouped 3x3 with >=16 channels per group.
WINOGRAD_CASES = [
    ((1, 32, 19, 21), 32, (3, 3), (1, 1), (1, 1), (1, 1), 2),
    ((2, 16, 8, 8), 16, (3, 3), (1, 1), (1, 1), (1, 1), 1),
]


def pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def solve(x, w, b, go_fn, stride, padding, dilation, groups):
    xd, wd = x.double(), w.double()
    bd = None if b is None else b.double()
    y = F.conv2d(xd, wd, bd, stride, padding, dilation, groups)
    go = go_fn(y.shape)
    dx, dw, db = torch.ops.aten.convolution_backward(
        go.double(), xd, wd, [w.shape[0]], list(stride), list(padding), list(dilation), False, [0, 0],
        groups, [True, True, True])
    return go, y.float(), dx.float(), dw.float(), db.float()


def main():
    out = {}
    meta = []

    def add(tag, x, w, b, go, y, dx, dw, db, geom):
        i = len(meta)
        meta.append((tag,) + geom)
        for k, v in (("x", x), ("w", w), ("b", b), ("go", go), ("y", y), ("dx", dx), ("dw", dw), ("db", db)):
            if v is not None:
                out[f"c{i}_{k}"] = v.numpy().astype(np.float32)
        out[f"c{i}_geom"] = np.array([*x.shape, w.shape[0], *geom[0], *geom[1], *geom[2], *geom[3], geom[4]],
                                     dtype=np.int64)

    for xshape, cout, kernel, stride, padding, dilation, groups in DISPATCH_CASES + WINOGRAD_CASES:
        g = torch.Generator().manual_seed(813 + sum(xshape) + sum(kernel))
        x = torch.randn(xshape, generator=g) * 0.2
        w = torch.randn((cout, xshape[1] // groups, *kernel), generator=g) * 0.2
        b = torch.randn((cout,), generator=g) * 0.2
        go, y, dx, dw, db = solve(x, w, b, lambda s: torch.randn(s, generator=g) * 0.3,
                                  stride, padding, dilation, groups)
        add("dispatch", x, w, b, go, y, dx, dw, db, (kernel, stride, padding, dilation, groups))

    for shape, channels, kernel, stride, padding, dilation, groups, bias in BASIC_CASES:
        torch.manual_seed(72)
        x = torch.randn(*shape)
        w = torch.randn(channels, shape[1] // groups, kernel, kernel)
        b = torch.randn(channels) if bias else None
        go, y, dx, dw, db = solve(x, w, b, lambda s: torch.randn(s), pair(stride), pair(padding),
                                  pair(dilation), groups)
        add("basic", x, w, b, go, y, dx, dw, db, (pair(kernel), pair(stride), pair(padding), pair(dilation), groups))

    for xshape, cout, kernel, stride, padding, dilation, groups in UNIVERSAL_CASES:
        torch.manual_seed(sum(xshape) + cout + sum(kernel))
        x = torch.randn(*xshape)
        w = torch.randn(cout, xshape[1] // groups, *kernel)
        b = torch.randn(cout)
        go, y, dx, dw, db = solve(x, w, b, lambda s: torch.randn(s), stride, padding, dilation, groups)
        add("universal", x, w, b, go, y, dx, dw, db, (kernel, stride, padding, dilation, groups))

    # A scaled-down slice of the headline single-layer configuration (N=8,C=64,56x56,
    # 3x3 pad 1, nn.Conv2d default init, seed 0), kept small enough to commit.
    torch.manual_seed(0)
    conv = torch.nn.Conv2d(64, 64, 3, padding=1)
    x = torch.randn(1, 64, 12, 12)
    go, y, dx, dw, db = solve(x, conv.weight.detach(), conv.bias.detach(), lambda s: torch.randn(s),
                              (1, 1), (1, 1), (1, 1), 1)
    add("layer64", x, conv.weight.detach(), conv.bias.detach(), go, y, dx, dw, db,
        ((3, 3), (1, 1), (1, 1), (1, 1), 1))

    out["tags"] = np.array([m[0] for m in meta])
    np.savez_compressed(os.path.join(HERE, "conv_cases.npz"), **out)

    # GEMM / addmm: shapes of tests/test_fused_addmm.py:7-34 and tests/test_direct_mm_out.py:7-58
    gm = {}
    shapes = [(2, 3, 4), (17, 33, 9), (64, 64, 64), (130, 70, 96), (5, 1, 7)]
    for i, (M, K, N) in enumerate(shapes):
        g = torch.Generator().manual_seed(4100 + i)
        a = torch.randn(M, K, generator=g)
        bt = torch.randn(N, K, generator=g)  # consumed transposed (stride-swapped view)
        bias = torch.randn(N, generator=g)
        for j, (beta, alpha) in enumerate([(1.0, 1.0), (0.0, 1.0), (0.5, -2.0)]):
            ref = torch.addmm(bias.double(), a.double(), bt.t().double(), beta=beta, alpha=alpha).float()
            gm[f"g{i}_{j}_out"] = ref.numpy()
        gm[f"g{i}_a"], gm[f"g{i}_bt"], gm[f"g{i}_bias"] = a.numpy(), bt.numpy(), bias.numpy()
    gm["count"] = np.array(len(shapes))
    np.savez_compressed(os.path.join(HERE, "gemm_cases.npz"), **gm)
    print("cases:", len(meta), "bytes:", os.path.getsize(os.path.join(HERE, "conv_cases.npz")),
          os.path.getsize(os.path.join(HERE, "gemm_cases.npz")))


if __name__ == "__main__":
    main()
