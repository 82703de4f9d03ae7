"""CPU restatement of the reference's generic N-d convolution (TEST INFRASTRUCTURE ONLY: imported by tests/ and
nothing else; the product path never touches it).

The reference computes every convolution that is not a plain FP32 Conv2D with one generic shader
(csrc/shaders/convolution_nd.comp, host side csrc/ops/convolution_nd.cpp:51-74): 1 to 3 spatial dimensions, ordinary or
transposed, groups, mode 0 forward / 1 dInput / 2 dWeight / 3 dBias, and an int64 forward twin
(csrc/shaders/convolution_nd_int64.comp).  Here the same sums are written as one numpy contraction per filter tap, in
float64 (or int64 with wrapping arithmetic, which is what the integer shader's adds and multiplies do).

Pinned in tests/test_convnd_oracle.py against PyTorch's CPU convolutions on the cases of the reference's own test
(tests/test_complete_spatial_recurrent.py:7-48, which compares the device result with exactly those CPU operators).
"""
import itertools

import numpy as np


def _triple(v, rank, fill):
    v = [v] * rank if isinstance(v, int) else list(v)
    assert len(v) == rank
    return [fill] * (3 - rank) + v


def _lift(a, rank):
    """[n, c, spatial...] -> [n, c, d, h, w] with missing leading extents 1 (convolution_nd.cpp:24,26-37)."""
    return a.reshape(a.shape[:2] + (1,) * (3 - rank) + a.shape[2:])


def output_shape(xshape, wshape, stride, padding, dilation, output_padding, transposed, groups):
    """Result shape; the formulas of `geometry` (convolution_nd.cpp:33-35)."""
    rank = len(xshape) - 2
    s, p, d = _triple(stride, rank, 1)[3 - rank:], _triple(padding, rank, 0)[3 - rank:], _triple(dilation, rank, 1)[3 - rank:]
    op = _triple(output_padding, rank, 0)[3 - rank:]
    cout = wshape[1] * groups if transposed else wshape[0]
    out = []
    for a in range(rank):
        eff = (wshape[a + 2] - 1) * d[a] + 1
        out.append((xshape[a + 2] - 1) * s[a] - 2 * p[a] + eff + op[a] if transposed else (xshape[a + 2] + 2 * p[a] - eff) // s[a] + 1)
    return (xshape[0], cout) + tuple(out)


def _gather(src, wt, out_sp, s, p, d, groups, acc_dtype):
    """out[n, co, o] = sum_{ci, k} src[n, ci, o*s - p + k*d] * wt[co, ci_local, k]   (shader mode 0, ordinary)."""
    n, cin = src.shape[:2]
    cout, cig = wt.shape[:2]
    cog = cout // groups
    k = wt.shape[2:]
    pad = [(0, 0), (0, 0)] + [(p[a], p[a] + s[a]) for a in range(3)]  # slack so every strided window exists
    sp = np.pad(src.astype(acc_dtype), pad)
    out = np.zeros((n, cout) + tuple(out_sp), acc_dtype)
    for t in itertools.product(*(range(e) for e in k)):
        win = tuple(slice(t[a] * d[a], t[a] * d[a] + (out_sp[a] - 1) * s[a] + 1, s[a]) for a in range(3))
        xs = sp[(slice(None), slice(None)) + win]
        for g in range(groups):
            out[:, g * cog:(g + 1) * cog] += np.einsum("ncdhw,oc->nodhw", xs[:, g * cig:(g + 1) * cig],
                                                       wt[g * cog:(g + 1) * cog, :, t[0], t[1], t[2]].astype(acc_dtype))
    return out


def _scatter(src, wt, out_sp, s, p, d, groups, acc_dtype):
    """out[n, c2, i*s - p + k*d] += src[n, c1, i] * wt[c1, c2_local, k]   (shader mode 0, transposed)."""
    n, c1 = src.shape[:2]
    c1g = c1 // groups
    c2g = wt.shape[1]
    k = wt.shape[2:]
    in_sp = src.shape[2:]
    full = [(in_sp[a] - 1) * s[a] + (k[a] - 1) * d[a] + 1 for a in range(3)]
    full = [max(full[a], p[a] + out_sp[a]) for a in range(3)]       # room for the output padding
    out = np.zeros((n, c2g * groups) + tuple(full), acc_dtype)
    srca = src.astype(acc_dtype)
    for t in itertools.product(*(range(e) for e in k)):
        win = tuple(slice(t[a] * d[a], t[a] * d[a] + (in_sp[a] - 1) * s[a] + 1, s[a]) for a in range(3))
        for g in range(groups):
            out[(slice(None), slice(g * c2g, (g + 1) * c2g)) + win] += np.einsum(
                "ncdhw,co->nodhw", srca[:, g * c1g:(g + 1) * c1g], wt[g * c1g:(g + 1) * c1g, :, t[0], t[1], t[2]].astype(acc_dtype))
    crop = tuple(slice(p[a], p[a] + out_sp[a]) for a in range(3))
    return out[(slice(None), slice(None)) + crop]


def _pair_weight(a_walk, b_other, kshape, s, p, d, groups, acc_dtype):
    """dw[a, b_local, k] = sum_{n, o} walk[n, a, o] * other[n, b, o*s - p + k*d]   (shader mode 2)."""
    n, cw = a_walk.shape[:2]
    co = b_other.shape[1]
    cwg, cog = cw // groups, co // groups
    walk_sp = a_walk.shape[2:]
    pad = [(0, 0), (0, 0)] + [(p[a], p[a] + s[a] + (kshape[a] - 1) * d[a]) for a in range(3)]
    op = np.pad(b_other.astype(acc_dtype), pad)
    aw = a_walk.astype(acc_dtype)
    out = np.zeros((cw, cog) + tuple(kshape), acc_dtype)
    for t in itertools.product(*(range(e) for e in kshape)):
        win = tuple(slice(t[a] * d[a], t[a] * d[a] + (walk_sp[a] - 1) * s[a] + 1, s[a]) for a in range(3))
        os_ = op[(slice(None), slice(None)) + win]
        for g in range(groups):
            out[g * cwg:(g + 1) * cwg, :, t[0], t[1], t[2]] = np.einsum("nadhw,nbdhw->ab", aw[:, g * cwg:(g + 1) * cwg],
                                                                        os_[:, g * cog:(g + 1) * cog])
    return out


def forward(x, w, b=None, stride=1, padding=0, dilation=1, output_padding=0, transposed=False, groups=1):
    """Shader mode 0 (float64 accumulate for float input; wrapping int64 for integer input)."""
    rank = x.ndim - 2
    acc = np.int64 if x.dtype == np.int64 else np.float64
    s, p, d = _triple(stride, rank, 1), _triple(padding, rank, 0), _triple(dilation, rank, 1)
    shape = output_shape(x.shape, w.shape, stride, padding, dilation, output_padding, transposed, groups)
    out_sp = _lift(np.empty(shape, np.int8), rank).shape[2:]
    x5, w5 = _lift(x, rank), _lift(w, rank)
    with np.errstate(over="ignore"):
        y = (_scatter if transposed else _gather)(x5, w5, out_sp, s, p, d, groups, acc)
        if b is not None:
            y = y + np.asarray(b, acc).reshape(1, -1, 1, 1, 1)
    return y.reshape(shape)


def backward(grad, x, w, stride=1, padding=0, dilation=1, output_padding=0, transposed=False, groups=1):
    """Shader modes 1, 2, 3 in float64: (dx, dw, db)."""
    rank = x.ndim - 2
    s, p, d = _triple(stride, rank, 1), _triple(padding, rank, 0), _triple(dilation, rank, 1)
    g5, x5, w5 = _lift(grad, rank), _lift(x, rank), _lift(w, rank)
    if transposed:
        # y scatters x through w[ci, co_local, k]: dx gathers grad through the same taps (result channel ci contracts its
        # group's co), dw pairs x (walked) with grad (gathered)
        dx = _gather(g5, w5, x5.shape[2:], s, p, d, groups, np.float64)
        dw = _pair_weight(x5, g5, w5.shape[2:], s, p, d, groups, np.float64)
    else:
        # y gathers x through w[co, ci_local, k]: dx scatters grad through them, dw pairs grad (walked) with x (gathered)
        dx = _scatter(g5, w5, x5.shape[2:], s, p, d, groups, np.float64)
        dw = _pair_weight(g5, x5, w5.shape[2:], s, p, d, groups, np.float64)
    db = g5.astype(np.float64).sum(axis=(0, 2, 3, 4))
    return dx.reshape(x.shape), dw.reshape(w.shape), db
