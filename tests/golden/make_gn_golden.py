"""Generate the committed golden vectors for GroupNorm forward / backward.

Run here (CPU only):  python tests/golden/make_gn_golden.py

The reference stores no numeric fixtures for GroupNorm: tests/test_native_group_norm.py of the
reference draws seeded CPU tensors (seed 1000 + sum(shape) + groups, :20-21) and compares the device
result with PyTorch's CPU group norm.  This script makes the same draws for the same shapes and
stores inputs with the PyTorch-CPU FP64 results of `native_group_norm` and its backward.

Output: tests/golden/group_norm_cases.npz (about 60 KB).
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
# (shape, groups) of tests/test_native_group_norm.py:9-17, plus one block with two channels per group
# and planes off the vector width
CASES = [((2, 8, 4, 5), 4), ((1, 8, 8, 8), 1), ((1, 12, 3, 7), 3), ((2, 16, 8), 8), ((2, 8, 2, 3, 4), 2), ((1, 8, 2, 2), 8),
         ((2, 4, 1, 1), 2), ((3, 10, 9, 7), 5)]


def main():
    out, tags = {}, []
    for shape, groups in CASES:
        for affine in (False, True):
            torch.manual_seed(1000 + sum(shape) + groups)
            x = torch.randn(*shape)
            c = shape[1]
            w = torch.randn(c) if affine else None
            b = torch.randn(c) if affine else None
            g = torch.randn(*shape)
            n, hw = shape[0], int(np.prod(shape[2:]))
            d = lambda t: None if t is None else t.double()
            y, mean, rstd = torch.ops.aten.native_group_norm(d(x), d(w), d(b), n, c, hw, groups, 1e-5)
            # without affine parameters the gradients a weight of ones would get are still defined: store them
            wb = d(w) if affine else torch.ones(c, dtype=torch.float64)
            dx, dw, db = torch.ops.aten.native_group_norm_backward(d(g), d(x), mean, rstd, wb, n, c, hw, groups, [True] * 3)
            i = len(tags)
            tags.append("affine" if affine else "plain")
            out[f"c{i}_groups"] = np.array(groups)
            for k, v in dict(x=x, g=g, w=w, b=b, y=y, mean=mean, rstd=rstd, dx=dx, dw=dw, db=db).items():
                if v is not None:
                    out[f"c{i}_{k}"] = v.numpy()
    out["tags"] = np.array(tags)
    np.savez_compressed(os.path.join(HERE, "group_norm_cases.npz"), **out)
    print(len(tags), "cases")


if __name__ == "__main__":
    main()
