"""Generate the committed golden vectors for BatchNorm forward / backward.

Run here (CPU only):  python tests/golden/make_bn_golden.py

The reference stores no numeric fixtures for BatchNorm: tests/test_batch_norm.py of the reference
draws seeded CPU tensors and compares the device result with PyTorch's CPU
`native_batch_norm` / `native_batch_norm_backward`, in FP32 (:24-46) or promoted to FP64 for the
precision cases (:99-141).  This script makes the same kind of draws (same seeds, shapes,
momentum and eps as those tests) and stores the inputs with the PyTorch-CPU FP64 results, so that
the oracle and the CUDA path are checked against the reference's own ground truth.

Output: tests/golden/batch_norm_cases.npz (about 400 KB).
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# shapes of tests/test_batch_norm.py:19-23 (seed 90, momentum .23, eps 1e-4) x the four
# (training, affine, running statistics) rows of :25
NATIVE_SHAPES = [(7, 5), (2, 3, 11), (2, 5, 7, 9), (2, 3, 4, 5, 7), (3, 2, 4, 7), (2, 3, 2, 3, 2, 2)]
MODES = [(True, True, True), (True, False, False), (False, True, True), (False, False, True)]
# (shape, offset, noise, eps, affine) rows of :144-164: pairs, constants, high offsets, short reductions
PRECISION = [
    ((2, 3), 10000.0, .1, 1e-5, True), ((2, 3), 10000.0, .1, 0.0, False), ((2, 3), 1.0, 1e-4, 1e-5, False),
    ((2, 3), 1.0, 1e-4, 0.0, True), ((2, 3), 3.0, 0.0, 1e-5, True), ((2, 3), 3.0, 0.0, 0.0, False),
    ((1, 3, 1, 2), 10000.0, .1, 1e-5, True), ((1, 3, 2, 1), 1.0, 1e-4, 1e-5, False),
    ((1, 3, 1, 2), 3.0, 0.0, 1e-5, True),
    *[((1, 3, samples), 10000.0, .1, eps, True) for samples in (3, 8, 129) for eps in (0.0, 1e-5)],
    ((4, 3, 31, 19), 10000.0, .1, 1e-5, False),   # :62-71 stable variance
]


def run(x, g, w, b, rm, rv, training, momentum, eps):
    d = lambda t: None if t is None else t.double()
    rmd, rvd = (None if rm is None else rm.double().clone()), (None if rv is None else rv.double().clone())
    y, mean, inv = torch.ops.aten.native_batch_norm(d(x), d(w), d(b), rmd, rvd, training, momentum, eps)
    dx, dw, db = torch.ops.aten.native_batch_norm_backward(d(g), d(x), d(w), d(rm), d(rv), mean, inv, training, eps,
                                                           [True, True, True])
    return dict(y=y, mean=mean, inv=inv, dx=dx, dw=dw, db=db, rm_out=rmd, rv_out=rvd)


def main():
    out, tags = {}, []

    def store(tag, x, g, w, b, rm, rv, training, momentum, eps):
        i = len(tags)
        tags.append(tag)
        out[f"c{i}_cfg"] = np.array([float(training), momentum, eps], np.float64)
        for k, v in dict(x=x, g=g, w=w, b=b, rm=rm, rv=rv).items():
            if v is not None:
                out[f"c{i}_{k}"] = v.numpy()
        for k, v in run(x, g, w, b, rm, rv, training, momentum, eps).items():
            if v is not None:
                out[f"c{i}_{k}"] = v.numpy()

    for shape in NATIVE_SHAPES:
        for training, affine, stats in MODES:
            torch.manual_seed(90)
            x, g, c = torch.randn(shape), torch.randn(shape), shape[1]
            w = torch.randn(c) if affine else None
            b = torch.randn(c) if affine else None
            rm = torch.randn(c) if stats else None
            rv = torch.rand(c) + .3 if stats else None
            store("native", x, g, w, b, rm, rv, training, .23, 1e-4)
    for shape, offset, noise, eps, affine in PRECISION:
        gen = torch.Generator().manual_seed(397 + sum(shape))
        x = torch.randn(shape, generator=gen) * noise + offset
        g = torch.randn(shape, generator=gen) * 0.3
        c = shape[1]
        w = torch.linspace(-1.3, 1.7, c) if affine else None
        b = torch.linspace(-0.4, 0.2, c) if affine else None
        store("precision", x, g, w, b, torch.linspace(-3.0, 7.0, c), torch.linspace(0.7, 2.1, c), True, .23, eps)
    out["tags"] = np.array(tags)
    np.savez_compressed(os.path.join(HERE, "batch_norm_cases.npz"), **out)
    print(len(tags), "cases")


if __name__ == "__main__":
    main()
