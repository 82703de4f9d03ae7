#!/usr/bin/env python
"""Benchmark of the FP32 Conv2D hot path (forward + dInput + dWeight) on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N=1): the ResNet-50-style layer sweep, batch 64: 3x3 pad-1 layers
(64,64,56) (128,128,28) (256,256,14) (512,512,7), a 1x1 256->64 @56 and a 3x3 stride-2
128->128 56->28, each in NCHW and in channels-last, forward + dInput + dWeight per layer.
One "step" is one pass over all 12 layer instances.  Inputs are seeded synthetic tensors
(N(0,1) activations, kaiming-uniform weights) and stay resident in HBM for `value`; the
`e2e` figure repeats the step through the C-ABI with pinned HOST buffers, host->device and
device->host copies inside the timed region (uploads, kernels and downloads pipelined on three streams).  The working set of a step (about 1.7 GB) is
far larger than L2, so no explicit L2 flush is needed between iterations.

N>1 (torchrun, one rank per GPU): every rank runs the same sweep on its own batch of 64
(weak scaling, global batch 64*N) and the weight gradients of each layer are summed over
ranks with ONE NCCL all-reduce per step (all layers' dW in a single fused buffer) on the compute stream.

Prints ONE JSON line.  `--impl reference` times the reference's CPU path instead (PyTorch's CPU
convolution, which is what the reference falls back to and tests against) on a bounded sample.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "pytorch-vulkan_b200"))

BATCH = 64
# (cin, cout, hw, kernel, stride, padding)
LAYERS = [
    (64, 64, 56, 3, 1, 1),
    (128, 128, 28, 3, 1, 1),
    (256, 256, 14, 3, 1, 1),
    (512, 512, 7, 3, 1, 1),
    (256, 64, 56, 1, 1, 0),
    (128, 128, 56, 3, 2, 1),
]
WORKLOAD = "resnet50-style layer sweep, batch 64, 6 layers x {NCHW, channels-last}, fwd+dInput+dWeight, FP32"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def layer_flops(cin, cout, hw, k, s, p, batch=BATCH):
    oh = (hw + 2 * p - k) // s + 1
    return 2 * batch * oh * oh * cout * cin * k * k


# ------------------------------------------------------------------------------------------
# reference arm: the reference's CPU path for this operator (PyTorch CPU FP32 convolution)
# ------------------------------------------------------------------------------------------
def cpu_sample(steps, warmup):
    """Time fwd + backward(all) of a bounded sample of the sweep on the host cores.
    Sample: every layer of the sweep in NCHW at batch 4 (1/16 of the workload's batch)."""
    import torch
    import torch.nn.functional as F
    from oracle import oracle  # noqa: F401  (the CPU leg is the oracle's PyTorch layer)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sample_batch = 4
    cases, flops = [], 0
    g = torch.Generator().manual_seed(1000)
    for (cin, cout, hw, k, s, p) in LAYERS:
        x = torch.randn(sample_batch, cin, hw, hw, generator=g)
        w = (torch.rand(cout, cin, k, k, generator=g) * 2 - 1) / (cin * k * k) ** 0.5
        oh = (hw + 2 * p - k) // s + 1
        go = torch.randn(sample_batch, cout, oh, oh, generator=g)
        cases.append((x, w, go, s, p))
        flops += 3 * layer_flops(cin, cout, hw, k, s, p, sample_batch)

    def step():
        for x, w, go, s, p in cases:
            F.conv2d(x, w, None, s, p)
            torch.ops.aten.convolution_backward(go, x, w, None, [s, s], [p, p], [1, 1], False, [0, 0], 1,
                                                [True, True, False])
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=threads, kind="port",
                sample=f"all 6 sweep layers, NCHW, batch {sample_batch} (1/16 of the batch), PyTorch CPU FP32 "
                       f"conv2d + convolution_backward (the reference's CPU fallback and test ground truth), "
                       f"{steps} steps", ms_per_step=dt * 1e3)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 20))
    base = cpu_sample(steps, max(1, min(args.warmup, 3)))
    line = {"impl": "reference", "metric": "conv2d_fwd_bwd_tflops", "value": base["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": max(1, min(args.warmup, 3)),
            "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "l2": "inputs larger than L2"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# B200 arm
# ------------------------------------------------------------------------------------------
class Layer:
    def __init__(self, torch, b200conv, spec, channels_last, seed, device):
        cin, cout, hw, k, s, p = spec
        self.spec, self.channels_last = spec, channels_last
        self.p = b200conv.geometry((BATCH, cin, hw, hw), cout, (k, k), (s, s), (p, p))
        g = torch.Generator().manual_seed(seed)
        fmt = torch.channels_last if channels_last else torch.contiguous_format
        # host (pinned) copies for the end-to-end leg; device copies for the resident leg
        self.hx = torch.randn(BATCH, cin, hw, hw, generator=g).contiguous(memory_format=fmt).pin_memory()
        bound = 1.0 / (cin * k * k) ** 0.5  # kaiming_uniform(a=sqrt(5)) bound
        self.hw_ = ((torch.rand(cout, cin, k, k, generator=g) * 2 - 1) * bound).pin_memory()
        self.hgo = torch.randn(BATCH, cout, self.p.oh, self.p.ow, generator=g).contiguous(memory_format=fmt).pin_memory()
        self.x, self.w, self.go = self.hx.to(device), self.hw_.to(device), self.hgo.to(device)
        self.y = torch.empty(BATCH, cout, self.p.oh, self.p.ow, device=device)
        self.dx = torch.empty(BATCH, cin, hw, hw, device=device)
        self.dw = None  # a view into the step's fused gradient buffer (set by main)
        self.w_shape = (cout, cin, k, k)
        self.hy, self.hdx = (torch.empty(t.shape).pin_memory() for t in (self.y, self.dx))
        self.hdw = torch.empty(self.w_shape).pin_memory()
        self.flops = 3 * self.p.flops()
        # scratch budget per call: 512 MiB (the operator's default is 64 MiB; Winograd chunks less with more)
        self.ws_bytes = max(b200conv.workspace_bytes(self.p, ph, budget=512 << 20) for ph in (0, 1, 2))
        self.h2d = sum(t.numel() * 4 for t in (self.hx, self.hw_, self.hgo))
        self.d2h = sum(t.numel() * 4 for t in (self.hy, self.hdx, self.hdw))

    def views(self, b200conv):
        def v(t):
            return b200conv.View4(t.data_ptr(), (ctypes.c_int64 * 4)(*t.stride()))
        return v(self.x), v(self.w), v(self.go)


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in
# the strip-kernel summary under profiles/ (one layer of the sweep; bytes, not a live measurement)
NCU_TRAFFIC = {
    "tc_strip_dweight": {"bytes_per_launch": 53.7e6,
                         "note": "ncu, layer 128->128 28x28 3x3 batch 64 NCHW: 51.5 MB read + 2.2 MB written per "
                                 "launch against 51.9 MB algorithmic (x + dy + dW)"},
    "tc_strip_forward": {"bytes_per_launch": 26.9e6,
                         "note": "ncu, layer 128->128 28x28 3x3 batch 64: 26.9 MB read per launch (x + filter); the "
                                 "25.7 MB output was still in L2 when the capture ended"},
    "tc_strip_dinput": {"bytes_per_launch": 26.9e6,
                        "note": "ncu, layer 128->128 28x28 3x3 batch 64: 26.9 MB read per launch (dy + filter)"},
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--layers", default="", help="comma-separated layer indices (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import b200conv
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the convolution path has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    b200conv.init(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        # NCCL_DEBUG=VERSION makes NCCL print a banner on stdout, where only the JSON line belongs
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)
    L = b200conv.lib()
    stream = torch.cuda.current_stream().cuda_stream

    specs = LAYERS if not args.layers else [LAYERS[int(i)] for i in args.layers.split(",")]
    layers = []
    for i, spec in enumerate(specs):
        for cl in (False, True):
            layers.append(Layer(torch, b200conv, spec, cl, 1000 + 2 * i + int(cl) + 7919 * rank, device))
    ws_bytes = max(max(l.ws_bytes for l in layers), 1)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
    step_flops = sum(l.flops for l in layers)
    # all weight gradients of a step live in one buffer: the data-parallel exchange is ONE all-reduce
    grad_flat = torch.empty(sum(int(torch.tensor(l.w_shape).prod()) for l in layers), device=device)
    off = 0
    for l in layers:
        n = int(torch.tensor(l.w_shape).prod())
        l.dw = grad_flat[off:off + n].view(l.w_shape)
        off += n

    families = {}  # kernel family -> [flops, [event pairs]]

    def run_layer(l, timed):
        xv, wv, gv = l.views(b200conv)
        calls = (
            ("forward", lambda: L.b200_conv2d_forward(ctypes.byref(l.p), xv, wv, None, 0, l.y.data_ptr(),
                                                      ws.data_ptr(), ws_bytes, 0, stream)),
            ("dinput", lambda: L.b200_conv2d_dinput(ctypes.byref(l.p), gv, wv, l.dx.data_ptr(), ws.data_ptr(),
                                                    ws_bytes, 0, stream)),
            ("dweight", lambda: L.b200_conv2d_dweight(ctypes.byref(l.p), xv, gv, l.dw.data_ptr(), ws.data_ptr(),
                                                      ws_bytes, 0, stream)),
        )
        for name, fn in calls:
            if timed:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            b200conv.check(fn())
            if timed:
                e1.record()
                fam = families.setdefault(b200conv.last_kernel(), [0, []])
                fam[0] += l.p.flops()
                fam[1].append((e0, e1))

    def step(timed=False):
        for l in layers:
            run_layer(l, timed)
        if dist is not None:
            dist.all_reduce(grad_flat)  # data-parallel exchange: sum of the weight gradients

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = b200conv.launch_count()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        step(timed=True)
    t_end.record()
    barrier()
    launches = b200conv.launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    ms = t_start.elapsed_time(t_end) / args.steps
    status = b200conv.device_status()
    if status != 0:
        raise SystemExit(f"device status word is {status:#x}: a bounded wait gave up; numbers are invalid")

    # ---- end-to-end leg: host buffers in, host buffers out, copies inside the timed region ----
    # Three streams pipeline the step over its layers: uploads of layer i+1, compute of layer i and
    # downloads of layer i-1 overlap (PCIe is full duplex); events order the hand-offs, including the
    # reuse of each layer's device buffers by the next step.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in layers]
    ev_comp = [torch.cuda.Event() for _ in layers]
    ev_out = [torch.cuda.Event() for _ in layers]
    ev_grads = torch.cuda.Event()

    def e2e_step():
        for i, l in enumerate(layers):
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_comp[i])  # previous step's kernels have finished reading these inputs
                l.x.copy_(l.hx, non_blocking=True)
                l.w.copy_(l.hw_, non_blocking=True)
                l.go.copy_(l.hgo, non_blocking=True)
                ev_in[i].record(s_in)
            main.wait_event(ev_in[i])
            main.wait_event(ev_out[i])      # previous step's downloads of y/dx/dw have left the buffers
            run_layer(l, False)
            ev_comp[i].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[i])
                l.hy.copy_(l.y, non_blocking=True)
                l.hdx.copy_(l.dx, non_blocking=True)
                if dist is None:
                    l.hdw.copy_(l.dw, non_blocking=True)
                ev_out[i].record(s_out)
        if dist is not None:
            dist.all_reduce(grad_flat)
            ev_grads.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_grads)
                for i, l in enumerate(layers):
                    l.hdw.copy_(l.dw, non_blocking=True)
                    ev_out[i].record(s_out)

    def e2e_join():
        main.wait_stream(s_in)
        main.wait_stream(s_out)
    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    e2e_join()
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    e_end.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_end) / e2e_steps

    times = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = (float(v) for v in times.cpu())

    if rank == 0:
        pk = peaks()
        fam_stats = {}
        for name, (fl, pairs) in families.items():
            t = sum(a.elapsed_time(b) for a, b in pairs)
            fam_stats[name] = dict(ms_per_step=t / args.steps, tflops=fl / (t * 1e-3) / 1e12 if t > 0 else 0.0,
                                   calls_per_step=len(pairs) // args.steps)
        dominant = max(fam_stats, key=lambda k: fam_stats[k]["ms_per_step"])
        tf32_peak = pk["bf16_sustained"] / 2.0  # kind::tf32 runs at half the dense bf16 rate
        ach = fam_stats[dominant]["tflops"]
        roofline = {"bound": "tensor", "kernel": dominant, "achieved": ach, "peak": tf32_peak, "unit": "TFLOP/s",
                    "frac": ach / tf32_peak, "frac_of_3xtf32_ceiling": ach / (tf32_peak / 3.0),
                    "traffic": NCU_TRAFFIC.get(dominant, {}).get("bytes_per_launch"),
                    "traffic_note": NCU_TRAFFIC.get(dominant, {}).get("note"),
                    "peak_source": f"{pk['source']}: sustained bf16 {pk['bf16_sustained']} TFLOP/s / 2 (TF32 rate); "
                                   "3xTF32 issues 3 TF32 passes per algorithmic MAC, ceiling = peak/3; with BF16 cross terms (forward, dInput, "
                                   "dWeight from 128 channels) one TF32 and one BF16 pass of equal duration, ceiling = peak/2",
                    "families": fam_stats}
        cpu = None if args.no_cpu else cpu_sample(3, 1)
        line = {
            "metric": "conv2d_fwd_bwd_tflops", "value": world * step_flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": BATCH * world, "parallelism": f"dp{world}",
                       "l2": "inputs larger than L2 (1.7 GB working set per step), no flush needed",
                       "numerics": "split-precision FP32 on tcgen05, FP32 accumulate: forward/dInput TF32 hi*hi + BF16 cross terms, "
                                   "dWeight the same from 128 input channels, else 3xTF32; FP32 FMA on the CUDA-core paths"},
            "clocks": clocks,
            "e2e": {"value": world * step_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": sum(l.h2d for l in layers), "d2h_bytes_per_step": sum(l.d2h for l in layers),
                    "ms_per_step": e2e_ms},
            "gpu_launches": int(launches),
            "roofline": roofline,
        }
        if cpu:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
