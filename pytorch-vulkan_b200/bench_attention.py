#!/usr/bin/env python
"""Times batched matrix products and scaled dot-product attention through the C ABI on one B200.

  python pytorch-vulkan_b200/bench_attention.py [--reps R] [--shapes heads,tokens,dim;...]

For each shape (self-attention: tokens x tokens scores, head dimension `dim`) four calls are timed with
CUDA events on the launching stream: the two products of the forward pass as plain b200_bmm calls
(Q K^T and P V), b200_attention_forward and b200_attention_backward.  FLOPs: 2*heads*tokens^2*dim per
product, two products forward, five backward.  One JSON line per row.
"""
import argparse
import json
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

DEFAULT_SHAPES = [(16, 1024, 64), (64, 1024, 64), (8, 4096, 64), (16, 4096, 40)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--shapes", default="")
    args = ap.parse_args()
    import torch
    import b200conv
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the attention path has no CPU fallback")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    b200conv.init(0)
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream
    shapes = DEFAULT_SHAPES if not args.shapes else [tuple(int(v) for v in s.split(",")) for s in args.shapes.split(";")]

    def timed(fn):
        for _ in range(2):
            b200conv.check(fn())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            b200conv.check(fn())
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.reps

    for heads, t, d in shapes:
        gen = torch.Generator(device=dev).manual_seed(heads + t + d)
        q, k, v, g = (torch.randn(heads, t, d, device=dev, generator=gen) for _ in range(4))
        out, lse = torch.empty(heads, t, d, device=dev), torch.empty(heads, t, device=dev)
        dq, dk, dv = (torch.empty(heads, t, d, device=dev) for _ in range(3))
        scores = torch.empty(heads, t, t, device=dev)
        n_f = L.b200_attention_workspace(heads, t, t, d, d, 0)
        n_b = L.b200_attention_workspace(heads, t, t, d, d, 1)
        ws = torch.empty(n_b, dtype=torch.uint8, device=dev)
        P = lambda x: x.data_ptr()
        scale = 1.0 / math.sqrt(d)
        product = 2.0 * heads * t * t * d
        calls = [
            ("bmm_q_kt", product, lambda: L.b200_bmm(heads, t, t, d, P(q), t * d, d, 1, P(k), t * d, 1, d, P(scores), 0, stream)),
            ("bmm_p_v", product, lambda: L.b200_bmm(heads, t, d, t, P(scores), t * t, t, 1, P(v), t * d, d, 1, P(out), 0, stream)),
            ("attention_forward", 2 * product, lambda: L.b200_attention_forward(heads, t, t, d, d, P(q), P(k), P(v), None, 0, scale, P(out),
                                                                                P(lse), P(ws), n_f, stream)),
            ("attention_backward", 5 * product, lambda: L.b200_attention_backward(heads, t, t, d, d, P(g), P(q), P(k), P(v), None, P(out),
                                                                                  P(lse), 0, scale, P(dq), P(dk), P(dv), P(ws), n_b, stream)),
        ]
        for name, flops, fn in calls:
            before = b200conv.launch_count()
            b200conv.check(fn())
            launches = b200conv.launch_count() - before
            ms = timed(fn)
            print(json.dumps({"op": name, "heads": heads, "tokens": t, "dim": d, "scores_mb": round(4e-6 * heads * t * t, 1),
                              "us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1), "gpu_launches": launches,
                              "kernels": b200conv.last_kernel()}), flush=True)
        del q, k, v, g, scores, ws


if __name__ == "__main__":
    main()
