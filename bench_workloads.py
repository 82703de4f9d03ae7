"""Per-layer workloads of bench.py (`--workload cfg3|cfg4|batch_norm|group_norm|attention|conv3d`).

Each prints one JSON line per row (the per-phase timing tables).  Everything is timed with CUDA events on the launching stream through the C ABI, one B200.
`cold` rows (and every cfg3 / cfg4 row) write a 256 MB buffer, larger than the 126 MB L2, before each timed
call; `warm` rows run the calls back to back.
"""
import ctypes
import json
import math
import os

FLUSH_BYTES = 256 << 20


class Timer:
    def __init__(self, torch, b200conv, device, reps):
        self.torch, self.b200conv, self.reps = torch, b200conv, reps
        self.flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=device)

    def time(self, fn, cold):
        torch, check = self.torch, self.b200conv.check
        for _ in range(3):
            check(fn())
        if not cold:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(self.reps):
                check(fn())
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / self.reps
        samples = []
        for _ in range(self.reps):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            check(fn())
            e1.record()
            torch.cuda.synchronize()
            samples.append(e0.elapsed_time(e1))
        samples.sort()
        return samples[len(samples) // 2]   # median

    def time_in_graph(self, fn_on):
        """`reps` calls captured into one CUDA graph and replayed: device time per call without the host's launch
        cost between calls.  fn_on(stream) issues the call on the given stream."""
        torch = self.torch
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            capture_stream = torch.cuda.current_stream().cuda_stream
            for _ in range(self.reps):
                self.b200conv.check(fn_on(capture_stream))
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / self.reps


# ---- configs 3 and 4 (U-Net block; grouped, dilated, strided, 1x1): every layer kind, every phase ----------------
CFG3 = [(32, c, c, hw, 3, dict(padding=(1, 1))) for c in (64, 128, 256, 512) for hw in (64, 32, 16, 33)]
CFG4 = [
    (16, 128, 128, 64, 3, dict(padding=(1, 1))), (16, 256, 256, 32, 3, dict(padding=(1, 1))), (16, 512, 512, 16, 3, dict(padding=(1, 1))),
    (16, 128, 128, 64, 3, dict(padding=(1, 1), groups=32)), (16, 256, 256, 32, 3, dict(padding=(1, 1), groups=32)),
    (16, 512, 512, 16, 3, dict(padding=(1, 1), groups=32)),
    (16, 128, 128, 64, 3, dict(padding=(2, 2), dilation=(2, 2))), (16, 256, 256, 32, 3, dict(padding=(2, 2), dilation=(2, 2))),
    (16, 128, 256, 64, 3, dict(stride=(2, 2), padding=(1, 1))), (16, 256, 512, 32, 3, dict(stride=(2, 2), padding=(1, 1))),
    (16, 128, 256, 64, 1, dict()), (16, 256, 512, 32, 1, dict()),
]


def _conv_rows(args, torch, b200conv, device, pk, name, specs, sliced_views):
    """forward, dInput, dWeight, dBias of each (n, cin, cout, hw, k, kwargs), NCHW and channels-last.  With
    sliced_views the input is the interior [:, 4:4+C, 1:1+H, 1:1+W] of a larger allocation (offset, non-dense strides),
    as config 4 states it."""
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream
    timer = Timer(torch, b200conv, device, args.reps)
    tf32_peak = pk["bf16_sustained"] / 2.0
    for n, cin, cout, hw, k, kw in specs:
        groups = kw.get("groups", 1)
        for cl in (False, True):
            gen = torch.Generator(device=device).manual_seed(n + cin + cout + hw + k)
            fmt = torch.channels_last if cl else torch.contiguous_format
            if sliced_views:
                base = torch.randn(n, cin + 8, hw + 2, hw + 2, device=device, generator=gen).contiguous(memory_format=fmt)
                x = base[:, 4:4 + cin, 1:1 + hw, 1:1 + hw]
            else:
                x = torch.randn(n, cin, hw, hw, device=device, generator=gen).contiguous(memory_format=fmt)
            p = b200conv.geometry((n, cin, hw, hw), cout, (k, k), kw.get("stride", (1, 1)), kw.get("padding", (0, 0)),
                                  kw.get("dilation", (1, 1)), groups)
            w = (torch.rand(cout, cin // groups, k, k, device=device, generator=gen) * 2 - 1) / math.sqrt(cin // groups * k * k)
            b = torch.randn(cout, device=device, generator=gen)
            go = torch.randn(n, cout, p.oh, p.ow, device=device, generator=gen).contiguous(memory_format=fmt)
            y, dx = torch.empty(n, cout, p.oh, p.ow, device=device), torch.empty(n, cin, hw, hw, device=device)
            dw, db = torch.empty_like(w), torch.empty(cout, device=device)
            ws_n = max(max(b200conv.workspace_bytes(p, ph, budget=512 << 20) for ph in range(4)), 1)
            ws = torch.empty(ws_n, dtype=torch.uint8, device=device)
            V = lambda t: b200conv.View4(t.data_ptr(), (ctypes.c_int64 * 4)(*t.stride()))
            xv, wv, gv = V(x), V(w), V(go)
            calls = {
                "forward": lambda: L.b200_conv2d_forward(ctypes.byref(p), xv, wv, b.data_ptr(), 1, y.data_ptr(), ws.data_ptr(), ws_n, 0, stream),
                "dinput": lambda: L.b200_conv2d_dinput(ctypes.byref(p), gv, wv, dx.data_ptr(), ws.data_ptr(), ws_n, 0, stream),
                "dweight": lambda: L.b200_conv2d_dweight(ctypes.byref(p), xv, gv, dw.data_ptr(), ws.data_ptr(), ws_n, 0, stream),
                "dbias": lambda: L.b200_conv2d_dbias(ctypes.byref(p), gv, db.data_ptr(), ws.data_ptr(), ws_n, stream),
            }
            flops = p.flops()
            nbytes = {"forward": 4 * (x.numel() + w.numel() + cout + y.numel()), "dinput": 4 * (go.numel() + w.numel() + dx.numel()),
                      "dweight": 4 * (x.numel() + go.numel() + dw.numel()), "dbias": 4 * (go.numel() + cout)}
            row = {"workload": name, "n": n, "cin": cin, "cout": cout, "hw": hw, "k": k, "layout": "channels-last" if cl else "nchw",
                   "view": "sliced" if sliced_views else "dense", **{kk: list(v) if isinstance(v, tuple) else v for kk, v in kw.items()}}
            for phase, fn in calls.items():
                ms = timer.time(fn, cold=True)
                t_roof = max(nbytes[phase] / (pk["hbm_gbs"] * 1e9), 0.0 if phase == "dbias" else flops / (tf32_peak * 1e12))
                row[phase] = {"us": round(ms * 1e3, 1), "kernel": b200conv.last_kernel(),
                              "tflops": None if phase == "dbias" else round(flops / ms / 1e9, 1),
                              "gbs": round(nbytes[phase] / ms / 1e6, 1),
                              "bound": "hbm" if nbytes[phase] / (pk["hbm_gbs"] * 1e9) >= (0.0 if phase == "dbias" else flops / (tf32_peak * 1e12)) else "tensor",
                              "frac_of_roofline": round(t_roof / (ms * 1e-3), 3)}
            print(json.dumps(row), flush=True)
            del x, go, y, dx, ws
    assert b200conv.device_status() == 0


def run_cfg3(args, torch, b200conv, device, pk):
    _conv_rows(args, torch, b200conv, device, pk, "cfg3", CFG3, sliced_views=False)


def run_cfg4(args, torch, b200conv, device, pk):
    _conv_rows(args, torch, b200conv, device, pk, "cfg4", CFG4, sliced_views=True)


# ---- BatchNorm -------------------------------------------------------------------------------------------------
BN_SHAPES = [(64, 64, 3136), (64, 256, 3136), (64, 128, 784), (64, 256, 196), (64, 512, 49), (64, 1024, 3136)]
BN_BYTES = {"train_forward": 12, "train_forward_add_relu": 16, "eval_forward": 8, "train_backward": 20}


def _shapes(args, default):
    return default if not args.shapes else [tuple(int(v) for v in s.split(",")) for s in args.shapes.split(";")]


def _cpu_norm_baseline(torch, kind, shape):
    """PyTorch CPU FP32 forward and backward of the operator on the host cores (the arithmetic the reference's
    tests compare with), best of four."""
    import time
    if kind == "batch_norm":
        n, c, s = shape
        groups = None
    else:
        n, c, s, groups = shape
    x, g = torch.randn(n, c, s), torch.randn(n, c, s)
    w, b, rm, rv = torch.randn(c), torch.randn(c), torch.zeros(c), torch.ones(c)
    saved = None
    for name in ("forward", "backward"):
        best = float("inf")
        for _ in range(4):
            t0 = time.perf_counter()
            if kind == "batch_norm" and name == "forward":
                saved = torch.ops.aten.native_batch_norm(x, w, b, rm, rv, True, 0.1, 1e-5)
            elif kind == "batch_norm":
                torch.ops.aten.native_batch_norm_backward(g, x, w, rm, rv, saved[1], saved[2], True, 1e-5, [True, True, True])
            elif name == "forward":
                saved = torch.ops.aten.native_group_norm(x, w, b, n, c, s, groups, 1e-5)
            else:
                torch.ops.aten.native_group_norm_backward(g, x, saved[1], saved[2], w, n, c, s, groups, [True, True, True])
            best = min(best, time.perf_counter() - t0)
        print(json.dumps({"workload": kind, "op": name, "shape": list(shape), "impl": "pytorch-cpu-fp32",
                          "cores": torch.get_num_threads(), "us": round(best * 1e6, 1)}), flush=True)


def run_batch_norm(args, torch, b200conv, device, pk):
    """Training forward (plain and with the fused residual add + ReLU), evaluation forward and training backward,
    planar (NCHW) and interleaved (channels-last), warm and cold.  Algorithmic bytes per element: 12 / 16 / 8 / 20."""
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream
    timer = Timer(torch, b200conv, device, args.reps)
    if args.cpu_baseline:
        _cpu_norm_baseline(torch, "batch_norm", _shapes(args, BN_SHAPES)[0])
    for n, c, s in _shapes(args, BN_SHAPES):
        for layout, layout_name in ((b200conv.BN_PLANAR, "planar"), (b200conv.BN_INTERLEAVED, "interleaved")):
            gen = torch.Generator(device=device).manual_seed(n + c + s)
            x = torch.randn(n * c * s, device=device, generator=gen)
            g = torch.randn(n * c * s, device=device, generator=gen)
            y, dx = torch.empty_like(x), torch.empty_like(x)
            w, b = torch.randn(c, device=device, generator=gen), torch.randn(c, device=device, generator=gen)
            rm, rv = torch.zeros(c, device=device), torch.ones(c, device=device)
            sm, si, dw, db = (torch.empty(c, device=device) for _ in range(4))
            ws_n = L.b200_batch_norm_workspace(n, c, s, layout)
            ws = torch.empty(ws_n, dtype=torch.uint8, device=device)
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
                nbytes = BN_BYTES[name] * n * c * s
                modes = [("warm", lambda: timer.time(fn, False)), ("cold", lambda: timer.time(fn, True))]
                if args.graph:
                    modes.append(("graph", lambda: timer.time_in_graph(fn)))
                for cache, measure in modes:
                    ms = measure()
                    gbs = nbytes / ms / 1e6
                    print(json.dumps({"workload": "batch_norm", "op": name, "n": n, "c": c, "s": s, "layout": layout_name,
                                      "tensor_mb": round(4e-6 * n * c * s, 1), "cache": cache, "us": round(ms * 1e3, 1),
                                      "gpu_launches": launches, "kernels": b200conv.last_kernel(),
                                      "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                                                   "frac": round(gbs / pk["hbm_gbs"], 3), "peak_source": pk["source"]}}), flush=True)
            del x, g, y, dx


# ---- GroupNorm -------------------------------------------------------------------------------------------------
GN_SHAPES = [(64, 256, 3136, 32), (32, 320, 4096, 32), (16, 256, 4096, 32), (16, 512, 1024, 32), (8, 128, 16384, 32),
             (16, 1280, 64, 32)]


def run_group_norm(args, torch, b200conv, device, pk):
    """Forward and backward (dx, dw, db) of diffusion-U-Net sized blocks.  Algorithmic bytes per element: 8 / 12."""
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream
    timer = Timer(torch, b200conv, device, args.reps)
    if args.cpu_baseline:
        _cpu_norm_baseline(torch, "group_norm", _shapes(args, GN_SHAPES)[2])
    for n, c, hw, groups in _shapes(args, GN_SHAPES):
        gen = torch.Generator(device=device).manual_seed(n + c + hw)
        x = torch.randn(n * c * hw, device=device, generator=gen)
        g = torch.randn(n * c * hw, device=device, generator=gen)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        w, b = torch.randn(c, device=device, generator=gen), torch.randn(c, device=device, generator=gen)
        mean, rstd = torch.empty(n * groups, device=device), torch.empty(n * groups, device=device)
        dw, db = torch.empty(c, device=device), torch.empty(c, device=device)
        ws_n = L.b200_group_norm_workspace(n, c, hw, groups)
        ws = torch.empty(ws_n, dtype=torch.uint8, device=device)
        P = lambda t: t.data_ptr()
        calls = {
            "forward": (8, lambda: L.b200_group_norm_forward(n, c, hw, groups, P(x), P(w), P(b), 1e-5, P(y), P(mean), P(rstd), stream)),
            "backward": (12, lambda: L.b200_group_norm_backward(n, c, hw, groups, P(g), P(x), P(mean), P(rstd), P(w), P(dx), P(dw), P(db),
                                                                P(ws), ws_n, stream)),
        }
        for name, (per_element, fn) in calls.items():
            before = b200conv.launch_count()
            b200conv.check(fn())
            launches = b200conv.launch_count() - before
            nbytes = per_element * n * c * hw
            for cold in (False, True):
                ms = timer.time(fn, cold)
                gbs = nbytes / ms / 1e6
                print(json.dumps({"workload": "group_norm", "op": name, "n": n, "c": c, "hw": hw, "groups": groups,
                                  "tensor_mb": round(4e-6 * n * c * hw, 1), "cache": "cold" if cold else "warm", "us": round(ms * 1e3, 1),
                                  "gpu_launches": launches, "kernels": b200conv.last_kernel(),
                                  "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                                               "frac": round(gbs / pk["hbm_gbs"], 3), "peak_source": pk["source"]}}), flush=True)
        del x, g, y, dx


# ---- batched products and attention ----------------------------------------------------------------------------
ATT_SHAPES = [(16, 1024, 64), (64, 1024, 64), (8, 4096, 64), (16, 4096, 40)]


def run_attention(args, torch, b200conv, device, pk):
    """Self-attention shapes (heads, tokens, head dimension): the two products of the forward pass as plain b200_bmm
    calls, b200_attention_forward and b200_attention_backward.  FLOPs: 2*heads*tokens^2*dim per product, two products
    forward, five backward."""
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream
    timer = Timer(torch, b200conv, device, args.reps)
    for heads, t, d in _shapes(args, ATT_SHAPES):
        gen = torch.Generator(device=device).manual_seed(heads + t + d)
        q, k, v, g = (torch.randn(heads, t, d, device=device, generator=gen) for _ in range(4))
        out, lse = torch.empty(heads, t, d, device=device), torch.empty(heads, t, device=device)
        dq, dk, dv = (torch.empty(heads, t, d, device=device) for _ in range(3))
        scores = torch.empty(heads, t, t, device=device)
        n_f = L.b200_attention_workspace(heads, t, t, d, d, 0)
        n_b = L.b200_attention_workspace(heads, t, t, d, d, 1)
        ws = torch.empty(n_b, dtype=torch.uint8, device=device)
        P = lambda x: x.data_ptr()
        scale = 1.0 / math.sqrt(d)
        product = 2.0 * heads * t * t * d
        calls = [
            ("bmm_q_kt", product, lambda: L.b200_bmm(heads, t, t, d, P(q), t * d, d, 1, P(k), t * d, 1, d, P(scores), 0, stream)),
            ("bmm_p_v", product, lambda: L.b200_bmm(heads, t, d, t, P(scores), t * t, t, 1, P(v), t * d, d, 1, P(out), 0, stream)),
            ("attention_forward", 2 * product, lambda: L.b200_attention_forward(heads, t, t, d, d, P(q), P(k), P(v), None, 0, 0, scale, 0.0, None, P(out),
                                                                                P(lse), P(ws), n_f, stream)),
            ("attention_backward", 5 * product, lambda: L.b200_attention_backward(heads, t, t, d, d, P(g), P(q), P(k), P(v), None, 0, P(out),
                                                                                  P(lse), 0, scale, 0.0, None, P(dq), P(dk), P(dv), None, P(ws), n_b,
                                                                                  stream)),
        ]
        for name, flops, fn in calls:
            before = b200conv.launch_count()
            b200conv.check(fn())
            launches = b200conv.launch_count() - before
            ms = timer.time(fn, cold=False)
            print(json.dumps({"workload": "attention", "op": name, "heads": heads, "tokens": t, "dim": d,
                              "scores_mb": round(4e-6 * heads * t * t, 1), "us": round(ms * 1e3, 1),
                              "tflops": round(flops / ms / 1e9, 1), "gpu_launches": launches, "kernels": b200conv.last_kernel()}), flush=True)
        del q, k, v, g, scores, ws


# ---- 3-D convolution: the decomposition over depth taps against the one-thread-per-output kernel ---------------------
CONV3D_SHAPES = [(4, 64, 16, 56), (2, 128, 8, 28), (1, 32, 32, 64)]   # (batch, channels, depth, height = width); 3x3x3, padding 1


def run_conv3d(args, torch, b200conv, device, pk):
    """b200_convnd_forward / _backward on video-sized 3-D layers, once through the decomposition onto the 2-D kernels and
    once with the generic kernel pinned (B200_CONV3D_GENERIC).  FLOPs: 2 * N * D * H * W * Cout * Cin * 27 per phase."""
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream
    for n, c, d, hw in _shapes(args, CONV3D_SHAPES):
        gen = torch.Generator(device=device).manual_seed(n + c + d + hw)
        x = torch.randn(n, c, d, hw, hw, device=device, generator=gen)
        w = torch.randn(c, c, 3, 3, 3, device=device, generator=gen) * 0.05
        p, yshape = b200conv.convnd_geometry(tuple(x.shape), tuple(w.shape), 1, 1, 1)
        y, g = torch.empty(yshape, device=device), torch.randn(yshape, device=device, generator=gen)
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        flops = 2.0 * y.numel() * c * 27
        P = lambda t: t.data_ptr()
        calls = [
            ("forward", lambda: L.b200_convnd_forward(ctypes.byref(p), P(x), P(w), None, P(y), 0, stream)),
            ("dinput", lambda: L.b200_convnd_backward(ctypes.byref(p), P(g), P(x), P(w), P(dx), None, None, stream)),
            ("dweight", lambda: L.b200_convnd_backward(ctypes.byref(p), P(g), P(x), P(w), None, P(dw), None, stream)),
        ]
        for path in ("decomposed", "generic"):
            if path == "generic":
                os.environ["B200_CONV3D_GENERIC"] = "1"
            else:
                os.environ.pop("B200_CONV3D_GENERIC", None)
            timer = Timer(torch, b200conv, device, args.reps if path == "decomposed" else 2)
            for name, fn in calls:
                before = b200conv.launch_count()
                b200conv.check(fn())
                launches = b200conv.launch_count() - before
                ms = timer.time(fn, cold=False)
                print(json.dumps({"workload": "conv3d", "path": path, "phase": name, "n": n, "channels": c, "depth": d, "hw": hw,
                                  "kernel": [3, 3, 3], "us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                                  "gpu_launches": launches}), flush=True)
        os.environ.pop("B200_CONV3D_GENERIC", None)
        del x, w, y, g, dx, dw
