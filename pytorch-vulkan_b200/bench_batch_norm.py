#!/usr/bin/env python
"""Times the BatchNorm kernels through the C ABI on one B200 and reports them against the HBM roofline.

  python pytorch-vulkan_b200/bench_batch_norm.py [--reps R] [--shapes n,c,s;n,c,s...]

Shapes default to the activations of the convolution benchmark's layer sweep (batch 64).  For each
shape and layout (planar = NCHW, interleaved = channels-last) three calls are timed with CUDA events
on the launching stream: training forward, evaluation forward, training backward (dx, dw, db).
Algorithmic bytes per element: training forward 12 (statistics read, normalisation read, write; 16 with
the fused residual add and ReLU, which reads one more tensor),
evaluation 8 (read, write), backward 20 (x and g read for the sums, x and g read again, dx written).
`cold` rows write a 256 MB buffer (larger than L2) before every timed call; `warm` rows run the
calls back to back, so tensors smaller than L2 are partly served from it; with --graph a third row
times the calls inside one CUDA graph, which removes the host's launch cost (about 17 us per call from
Python) that bounds the warm rows of small tensors.  One JSON line per row.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

DEFAULT_SHAPES = [(64, 64, 3136), (64, 256, 3136), (64, 128, 784), (64, 256, 196), (64, 512, 49), (64, 1024, 3136)]
BYTES_PER_ELEMENT = {"train_forward": 12, "train_forward_add_relu": 16, "eval_forward": 8, "train_backward": 20}


def hbm_peak():
    path = os.path.join(HERE, "..", "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--shapes", default="")
    ap.add_argument("--graph", action="store_true",
                    help="also time each call as `reps` launches inside one CUDA graph (no host launch cost between calls)")
    ap.add_argument("--cpu-baseline", action="store_true",
                    help="also time PyTorch's CPU FP32 batch norm (the arithmetic the reference's tests compare with) on the host cores")
    args = ap.parse_args()
    import torch
    import b200conv
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the BatchNorm path has no CPU fallback")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    b200conv.init(0)
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peak, peak_source = hbm_peak()
    shapes = DEFAULT_SHAPES if not args.shapes else [tuple(int(v) for v in s.split(",")) for s in args.shapes.split(";")]

    def timed(fn, cold):
        for _ in range(3):
            b200conv.check(fn())
        if not cold:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.reps):
                b200conv.check(fn())
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / args.reps
        total = 0.0
        for _ in range(args.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            b200conv.check(fn())
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / args.reps

    def timed_in_graph(fn):
        """`reps` calls captured into one CUDA graph and replayed: device time per call without the
        host's launch cost between calls."""
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            capture_stream = torch.cuda.current_stream().cuda_stream
            for _ in range(args.reps):
                b200conv.check(fn(capture_stream))
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.reps

    if args.cpu_baseline:
        import time
        n, c, s = shapes[0]
        x, g = torch.randn(n, c, s), torch.randn(n, c, s)
        w, b, rm, rv = torch.randn(c), torch.randn(c), torch.zeros(c), torch.ones(c)
        for name, k in (("train_forward", 3), ("train_backward", 3)):
            best = float("inf")
            for _ in range(k + 1):
                t0 = time.perf_counter()
                if name == "train_forward":
                    y, sm, si = torch.ops.aten.native_batch_norm(x, w, b, rm, rv, True, 0.1, 1e-5)
                else:
                    torch.ops.aten.native_batch_norm_backward(g, x, w, rm, rv, sm, si, True, 1e-5, [True, True, True])
                best = min(best, time.perf_counter() - t0)
            nbytes = BYTES_PER_ELEMENT[name] * n * c * s
            print(json.dumps({"op": name, "n": n, "c": c, "s": s, "impl": "pytorch-cpu-fp32", "cores": torch.get_num_threads(),
                              "us": round(best * 1e6, 1), "GB/s": round(nbytes / best / 1e9, 1)}), flush=True)
    for n, c, s in shapes:
        for layout, layout_name in ((b200conv.BN_PLANAR, "planar"), (b200conv.BN_INTERLEAVED, "interleaved")):
            gen = torch.Generator(device=dev).manual_seed(n + c + s)
            x = torch.randn(n * c * s, device=dev, generator=gen)
            g = torch.randn(n * c * s, device=dev, generator=gen)
            y, dx = torch.empty_like(x), torch.empty_like(x)
            w, b = torch.randn(c, device=dev, generator=gen), torch.randn(c, device=dev, generator=gen)
            rm, rv = torch.zeros(c, device=dev), torch.ones(c, device=dev)
            sm, si, dw, db = (torch.empty(c, device=dev) for _ in range(4))
            ws_n = L.b200_batch_norm_workspace(n, c, s, layout)
            ws = torch.empty(ws_n, dtype=torch.uint8, device=dev)
            P = lambda t: t.data_ptr()
            calls = {
                "train_forward": lambda st=stream: L.b200_batch_norm_forward(n, c, s, layout, P(x), P(w), 1, P(b), 1, P(rm), 1, P(rv), 1, 1,
                                                                   0.1, 1e-5, P(y), P(sm), P(si), P(ws), ws_n, st),
                "train_forward_add_relu": lambda st=stream: L.b200_batch_norm_forward_fused(n, c, s, layout, P(x), P(w), 1, P(b), 1, P(rm), 1,
                                                                                  P(rv), 1, 1, 0.1, 1e-5, P(g), 1, P(y), P(sm), P(si),
                                                                                  P(ws), ws_n, st),
                "eval_forward": lambda st=stream: L.b200_batch_norm_forward(n, c, s, layout, P(x), P(w), 1, P(b), 1, P(rm), 1, P(rv), 1, 0,
                                                                  0.1, 1e-5, P(y), P(sm), P(si), P(ws), ws_n, st),
                "train_backward": lambda st=stream: L.b200_batch_norm_backward(n, c, s, layout, P(g), P(x), P(w), 1, P(sm), 1, P(si), 1, 1,
                                                                     1e-5, P(dx), P(dw), P(db), P(ws), ws_n, st),
            }
            for name, fn in calls.items():
                before = b200conv.launch_count()
                b200conv.check(fn())
                launches = b200conv.launch_count() - before
                nbytes = BYTES_PER_ELEMENT[name] * n * c * s
                modes = [("warm", lambda: timed(fn, False)), ("cold", lambda: timed(fn, True))]
                if args.graph:
                    modes.append(("graph", lambda: timed_in_graph(fn)))
                for cache, measure in modes:
                    cold = cache == "cold"
                    ms = measure()
                    gbs = nbytes / ms / 1e6
                    print(json.dumps({"op": name, "n": n, "c": c, "s": s, "layout": layout_name, "tensor_mb": round(4e-6 * n * c * s, 1),
                                      "cache": cache, "us": round(ms * 1e3, 1), "gpu_launches": launches,
                                      "kernels": b200conv.last_kernel(),
                                      "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                                                   "frac": round(gbs / peak, 3), "peak_source": peak_source}}), flush=True)
            del x, g, y, dx


if __name__ == "__main__":
    main()
