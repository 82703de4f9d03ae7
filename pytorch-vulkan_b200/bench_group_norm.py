#!/usr/bin/env python
"""Times the GroupNorm kernels through the C ABI on one B200 and reports them against the HBM roofline.

  python pytorch-vulkan_b200/bench_group_norm.py [--reps R] [--shapes n,c,hw,groups;...]

Default shapes are diffusion-U-Net sized blocks (32 groups).  Forward and backward (dx, dw, db) are
timed with CUDA events on the launching stream.  Algorithmic bytes per element: forward 8 (one read,
one write: the second pass over a block is served by L2), backward 12 (x and dy read, dx written).
`cold` rows write a 256 MB buffer (larger than L2) before every timed call.  One JSON line per row.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

DEFAULT_SHAPES = [(64, 256, 3136, 32), (32, 320, 4096, 32), (16, 256, 4096, 32), (16, 512, 1024, 32), (8, 128, 16384, 32),
                  (16, 1280, 64, 32)]
BYTES_PER_ELEMENT = {"forward": 8, "backward": 12}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--shapes", default="")
    args = ap.parse_args()
    import torch
    import b200conv
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the GroupNorm path has no CPU fallback")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    b200conv.init(0)
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    path = os.path.join(HERE, "..", "MEASURED_PEAKS.json")
    peak, peak_source = (json.load(open(path))["hbm_gbs"], "measured") if os.path.exists(path) else (6650.0, "fallback")
    shapes = DEFAULT_SHAPES if not args.shapes else [tuple(int(v) for v in s.split(",")) for s in args.shapes.split(";")]

    def timed(fn, cold):
        for _ in range(3):
            b200conv.check(fn())
        total = 0.0
        if not cold:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.reps):
                b200conv.check(fn())
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / args.reps
        for _ in range(args.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            b200conv.check(fn())
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / args.reps

    for n, c, hw, groups in shapes:
        gen = torch.Generator(device=dev).manual_seed(n + c + hw)
        x = torch.randn(n * c * hw, device=dev, generator=gen)
        g = torch.randn(n * c * hw, device=dev, generator=gen)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        w, b = torch.randn(c, device=dev, generator=gen), torch.randn(c, device=dev, generator=gen)
        mean, rstd = torch.empty(n * groups, device=dev), torch.empty(n * groups, device=dev)
        dw, db = torch.empty(c, device=dev), torch.empty(c, device=dev)
        ws_n = L.b200_group_norm_workspace(n, c, hw, groups)
        ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
        P = lambda t: t.data_ptr()
        calls = {
            "forward": lambda: L.b200_group_norm_forward(n, c, hw, groups, P(x), P(w), P(b), 1e-5, P(y), P(mean), P(rstd), stream),
            "backward": lambda: L.b200_group_norm_backward(n, c, hw, groups, P(g), P(x), P(mean), P(rstd), P(w), P(dx), P(dw), P(db),
                                                          P(ws), ws_n, stream),
        }
        for name, fn in calls.items():
            before = b200conv.launch_count()
            b200conv.check(fn())
            launches = b200conv.launch_count() - before
            nbytes = BYTES_PER_ELEMENT[name] * n * c * hw
            for cold in (False, True):
                ms = timed(fn, cold)
                gbs = nbytes / ms / 1e6
                print(json.dumps({"op": name, "n": n, "c": c, "hw": hw, "groups": groups, "tensor_mb": round(4e-6 * n * c * hw, 1),
                                  "cache": "cold" if cold else "warm", "us": round(ms * 1e3, 1), "gpu_launches": launches,
                                  "kernels": b200conv.last_kernel(),
                                  "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                                               "frac": round(gbs / peak, 3), "peak_source": peak_source}}), flush=True)
        del x, g, y, dx


if __name__ == "__main__":
    main()
