"""Loader for the committed golden vectors (tests/golden/*.npz)."""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_CONV = None


def conv_cases():
    """List of dicts: tag, x, w, b (or None), go, y, dx, dw, db, and the geometry
    (kernel, stride, padding, dilation, groups) of each stored case."""
    global _CONV
    if _CONV is None:
        z = np.load(os.path.join(HERE, "golden", "conv_cases.npz"))
        tags = list(z["tags"])
        cases = []
        for i, tag in enumerate(tags):
            g = [int(v) for v in z[f"c{i}_geom"]]
            case = dict(tag=str(tag), index=i, xshape=tuple(g[0:4]), cout=g[4], kernel=(g[5], g[6]),
                        stride=(g[7], g[8]), padding=(g[9], g[10]), dilation=(g[11], g[12]), groups=g[13])
            for k in ("x", "w", "b", "go", "y", "dx", "dw", "db"):
                key = f"c{i}_{k}"
                case[k] = z[key] if key in z.files else None
            cases.append(case)
        _CONV = cases
    return _CONV


def case_id(case):
    return "%s%d-%s-k%dx%d-g%d" % (case["tag"], case["index"], "x".join(map(str, case["xshape"])),
                                  case["kernel"][0], case["kernel"][1], case["groups"])


def gemm_cases():
    z = np.load(os.path.join(HERE, "golden", "gemm_cases.npz"))
    out = []
    for i in range(int(z["count"])):
        out.append(dict(a=z[f"g{i}_a"], bt=z[f"g{i}_bt"], bias=z[f"g{i}_bias"],
                        outs=[z[f"g{i}_{j}_out"] for j in range(3)],
                        scalars=[(1.0, 1.0), (0.0, 1.0), (0.5, -2.0)]))
    return out


_BN = None


def batch_norm_cases():
    """List of dicts: tag, training, momentum, eps, inputs x, g, w, b, rm, rv (None where absent) and
    the PyTorch-CPU FP64 results y, mean, inv, dx, dw, db, rm_out, rv_out."""
    global _BN
    if _BN is None:
        z = np.load(os.path.join(HERE, "golden", "batch_norm_cases.npz"))
        cases = []
        for i, tag in enumerate(z["tags"]):
            training, momentum, eps = z[f"c{i}_cfg"]
            case = dict(tag=str(tag), index=i, training=bool(training), momentum=float(momentum), eps=float(eps))
            for k in ("x", "g", "w", "b", "rm", "rv", "y", "mean", "inv", "dx", "dw", "db", "rm_out", "rv_out"):
                key = f"c{i}_{k}"
                case[k] = z[key] if key in z.files else None
            cases.append(case)
        _BN = cases
    return _BN


def bn_case_id(case):
    return f"{case['tag']}{case['index']}-" + "x".join(map(str, case["x"].shape)) + ("-train" if case["training"] else "-eval")


_GN = None


def group_norm_cases():
    """List of dicts: tag, groups, inputs x, g, w, b (None where absent) and the PyTorch-CPU FP64
    results y, mean, rstd, dx, dw, db."""
    global _GN
    if _GN is None:
        z = np.load(os.path.join(HERE, "golden", "group_norm_cases.npz"))
        cases = []
        for i, tag in enumerate(z["tags"]):
            case = dict(tag=str(tag), index=i, groups=int(z[f"c{i}_groups"]))
            for k in ("x", "g", "w", "b", "y", "mean", "rstd", "dx", "dw", "db"):
                key = f"c{i}_{k}"
                case[k] = z[key] if key in z.files else None
            cases.append(case)
        _GN = cases
    return _GN


def gn_case_id(case):
    return f"{case['tag']}{case['index']}-" + "x".join(map(str, case["x"].shape)) + f"-g{case['groups']}"
