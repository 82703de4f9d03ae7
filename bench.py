#!/usr/bin/env python
"""Benchmark of the FP32 Conv2D hot path (forward + dInput + dWeight) on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Default workload `sweep` (the one the headline metric is quoted on): the ResNet-50-style layer sweep,
batch 64: 3x3 pad-1 layers (64,64,56) (128,128,28) (256,256,14) (512,512,7), a 1x1 256->64 @56 and a 3x3
stride-2 128->128 56->28, each in NCHW and in channels-last, forward + dInput + dWeight per layer.  One
"step" is one pass over all 12 layer instances.  Inputs are seeded synthetic tensors (N(0,1) activations,
kaiming-uniform weights) and stay resident in HBM for `value`; the `e2e` figure repeats the step through
the C-ABI with pinned HOST buffers, host->device and device->host copies inside the timed region
(uploads, kernels and downloads pipelined on three streams).  The working set of a step (about 1.7 GB)
is far larger than L2, so no explicit L2 flush is needed between iterations.

The line also carries
  max_rel_err   the metric's third clause: max over the step's outputs of ||out - ref||_2 / ||ref||_2 against
                the PyTorch-CPU FP64 oracle, on a fixed sample of every layer (two images for y and dX, four
                output channels over the whole batch for dW), computed outside the timed region;
  config5       the sharded configuration: global batch 512 split evenly over the ranks, 256 -> 256 channels,
                56 x 56, per-sample seeds, forward + dWeight + dBias + dInput per step with the all-reduce of
                the fused dW || dB buffer (2.36 MB) issued through the library's communicator on a second
                stream under the dInput kernel; strong scaling (the driver compares ms_per_step over N).

The timed steps replay ONE CUDA graph of a step (its 72 kernel launches are recorded through the C ABI on the
benchmark's stream after the warm-up steps; `launch_mode` says so, `gpu_launches` counts the recorded launches
times the replays plus what is launched outside the graph); `--eager` issues every call separately instead.  The
per-family times of `roofline` come from an extra eager pass with events around every call, before the timed region.

N>1 (torchrun, one rank per GPU): every rank runs the same sweep on its own batch of 64 (weak scaling,
global batch 64*N); the dWeight kernels write into one fused gradient buffer (26 MB), which b200_allreduce_sum_f32
(NCCL behind the C ABI) sums over the ranks once per step after the last layer, on a second stream.
`--bucket-mb M` exchanges buckets of about M MB of consecutive layers under the following layers' kernels instead
(the step is then cut into one graph per bucket).  torch.distributed carries only the rendezvous, the barrier
and the max-over-ranks of the timings.

Other workloads (one JSON line per row: the per-layer, per-phase timing tables):
  cfg3 / cfg4   per-layer, per-phase times of the U-Net-block and ResNeXt/dilated/strided configurations (configs 3 and 4) (L2 flushed before every call)
  cfg5          config 5 alone
  batch_norm / group_norm / attention   the kernels of the rows next to the convolution
  conv3d        3-D layers through the depth-tap decomposition and through the generic kernel

`--impl reference` times the reference's CPU path (PyTorch's CPU convolution, which is what the reference
falls back to and tests against) on the same sweep.  `--layers`, `--no-cpu`, `--no-cfg5`, `--no-e2e` exist
for profiling runs (they shorten what runs under ncu) and are not part of the contract.
"""
import argparse
import ctypes
import json
import math
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
L2_NOTE = "inputs larger than L2 (1.7 GB working set per step), no flush needed"
NUMERICS = ("split-precision FP32 on tcgen05, FP32 accumulate: TF32 hi*hi + BF16 cross terms (dWeight: the same, "
            "or three TF32 passes where the plan says so); FP32 FMA on the CUDA-core paths")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples the SM clock and the throttle reasons while the timed region runs (read-only): NVML every 2 ms from a
    thread of this process where pynvml is importable, otherwise `nvidia-smi -lms 100`."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.nvml, self.running, self.counting = [], None, None, False, False
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in visible.split(",") if v.strip() != ""]
            phys = int(ids[index]) if ids and all(v.strip().isdigit() for v in ids) and index < len(ids) else index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.period = max(0.001, float(os.environ.get("B200_BENCH_CLOCK_PERIOD_MS", "2")) / 1000.0)
            self.running = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _poll(self):
        n = self.nvml
        bits = (("hw_slowdown", n.nvmlClocksThrottleReasonHwSlowdown), ("hw_thermal_slowdown", n.nvmlClocksThrottleReasonHwThermalSlowdown),
                ("sw_thermal_slowdown", n.nvmlClocksThrottleReasonSwThermalSlowdown), ("sw_power_cap", n.nvmlClocksThrottleReasonSwPowerCap))
        while self.running:
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                if self.counting:
                    self.rows.append([str(mhz), str(self.max_mhz)] + ["Active" if mask & bit else "Not Active" for _, bit in bits])
            except Exception:
                pass
            time.sleep(self.period)

    def _read(self):
        for line in self.proc.stdout:
            if self.counting:
                self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        """The timed region starts now: samples taken before this call (while the ranks met at the barrier) are not kept."""
        self.counting = True

    def stop(self):
        if self.nvml:
            self.running = False
            self.thread.join(timeout=1)
        elif not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        else:
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
                "reasons": reasons, "samples": len(sm), "sm_mhz_min": min(sm) if sm else None,
                "source": "nvml, 2 ms period" if self.nvml else "nvidia-smi, 100 ms period"}


def layer_flops(cin, cout, hw, k, s, p, batch=BATCH):
    oh = (hw + 2 * p - k) // s + 1
    return 2 * batch * oh * oh * cout * cin * k * k


def sweep_config(world):
    return {"workload": WORKLOAD, "global_batch": BATCH * world, "parallelism": f"dp{world}", "l2": L2_NOTE}


# ------------------------------------------------------------------------------------------
# the reference's CPU path for this operator: PyTorch CPU FP32 convolution on all host cores
# ------------------------------------------------------------------------------------------
def host_sweep_tensors(torch, specs, rank=0, pin=False):
    """(x, w, dy) of every layer instance of the sweep, NCHW and channels-last, seeded as the B200 arm seeds them."""
    out = []
    for i, (cin, cout, hw, k, s, p) in enumerate(specs):
        for cl in (False, True):
            g = torch.Generator().manual_seed(1000 + 2 * i + int(cl) + 7919 * rank)
            fmt = torch.channels_last if cl else torch.contiguous_format
            oh = (hw + 2 * p - k) // s + 1
            x = torch.randn(BATCH, cin, hw, hw, generator=g).contiguous(memory_format=fmt)
            w = (torch.rand(cout, cin, k, k, generator=g) * 2 - 1) / (cin * k * k) ** 0.5   # kaiming_uniform(a=sqrt(5))
            go = torch.randn(BATCH, cout, oh, oh, generator=g).contiguous(memory_format=fmt)
            if pin:
                x, w, go = x.pin_memory(), w.pin_memory(), go.pin_memory()
            out.append(((cin, cout, hw, k, s, p), cl, x, w, go))
    return out


def cpu_sweep(torch, tensors, steps, warmup):
    """fwd + backward(dX, dW) of every layer instance on the host cores: per-step seconds."""
    import torch.nn.functional as F
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)

    def step():
        for (cin, cout, hw, k, s, p), _, x, w, go in tensors:
            F.conv2d(x, w, None, s, p)
            torch.ops.aten.convolution_backward(go, x, w, None, [s, s], [p, p], [1, 1], False, [0, 0], 1,
                                                [True, True, False])
    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return times, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    tensors = host_sweep_tensors(torch, LAYERS)
    flops = sum(3 * layer_flops(*spec) for spec, *_ in tensors)
    times, threads = cpu_sweep(torch, tensors, args.steps, args.warmup)
    dt = sum(times) / len(times)
    value = flops / dt / 1e12
    line = {"impl": "reference", "metric": "conv2d_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": sweep_config(1),
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                             "sample": f"the full sweep (12 layer instances, batch 64, both layouts), {args.steps} steps after "
                                       f"{args.warmup} warm-ups, PyTorch CPU FP32 conv2d + convolution_backward "
                                       "(the reference's CPU fallback and its tests' ground truth)"},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# B200 arm
# ------------------------------------------------------------------------------------------
class Layer:
    def __init__(self, torch, b200conv, spec, channels_last, hx, hw_, hgo, device):
        cin, cout, hw, k, s, p = spec
        self.spec, self.channels_last = spec, channels_last
        self.p = b200conv.geometry((BATCH, cin, hw, hw), cout, (k, k), (s, s), (p, p))
        # host (pinned) copies for the end-to-end leg; device copies for the resident leg
        self.hx, self.hw_, self.hgo = hx, hw_, hgo
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


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the family's kernel on ONE layer of the sweep
# (named in the note), from the ncu capture summarised in the strip-kernel summary under profiles/: bytes of
# that capture, not a live measurement and not a figure for the whole family.
NCU_TRAFFIC_ONE_LAYER = {
    "tc_strip_dweight": {"bytes_per_launch": 54.4e6, "layer": "128->128 28x28 3x3 batch 64 NCHW",
                         "note": "51.5 MB read + 2.9 MB written per launch against 51.9 MB algorithmic (x + dy + dW)"},
    "tc_tstrip_forward": {"bytes_per_launch": 26.9e6, "layer": "128->128 28x28 3x3 batch 64 NCHW",
                          "note": "26.9 MB read per launch (x + filter); the 25.7 MB output was still in L2 when the capture ended"},
    "tc_tstrip_dinput": {"bytes_per_launch": 26.9e6, "layer": "128->128 28x28 3x3 batch 64 NCHW",
                         "note": "26.9 MB read per launch (dy + filter)"},
    "tc_strip_forward": {"bytes_per_launch": 26.9e6, "layer": "128->128 28x28 3x3 batch 64 NCHW",
                         "note": "26.9 MB read per launch (x + filter), pixels-on-M arrangement of the same layer"},
    "tc_strip_dinput": {"bytes_per_launch": 26.9e6, "layer": "128->128 28x28 3x3 batch 64 NCHW",
                        "note": "26.9 MB read per launch (dy + filter), pixels-on-M arrangement of the same layer"},
}


def rel_l2(torch, got, want):
    got, want = got.double().reshape(-1), want.double().reshape(-1)
    den = float(want.norm())
    return float((got - want).norm()) / den if den > 0 else float((got - want).norm())


def sampled_max_rel_err(torch, layers, check_dw):
    """max over layers and outputs of the relative L2 error against the PyTorch-CPU FP64 oracle on a fixed sample:
    images 0 and 63 for y and dX (independent per image), output channels {0, 1, mid, last} over the whole batch for dW
    (a row of dW depends on that channel of dy only)."""
    import torch.nn.functional as F
    worst, per_output = 0.0, {"y": 0.0, "dx": 0.0, "dw": 0.0}
    for l in layers:
        cin, cout, hw, k, s, p = l.spec
        idx = torch.tensor([0, BATCH - 1])
        x, w, go = l.hx.double(), l.hw_.double(), l.hgo.double()
        wy = F.conv2d(x[idx], w, None, s, p)
        wdx = torch.ops.aten.convolution_backward(go[idx], x[idx], w, None, [s, s], [p, p], [1, 1], False, [0, 0], 1,
                                                  [True, False, False])[0]
        errs = {"y": rel_l2(torch, l.y[idx.to(l.y.device)].cpu(), wy), "dx": rel_l2(torch, l.dx[idx.to(l.dx.device)].cpu(), wdx)}
        if check_dw:
            co = torch.tensor(sorted({0, 1, cout // 2, cout - 1}))
            wdw = torch.ops.aten.convolution_backward(go[:, co].contiguous(), x, w[co].contiguous(), None, [s, s], [p, p], [1, 1],
                                                      False, [0, 0], 1, [False, True, False])[1]
            errs["dw"] = rel_l2(torch, l.dw[co.to(l.dw.device)].cpu(), wdw)
        for k_, v in errs.items():
            per_output[k_] = max(per_output[k_], v)
        worst = max(worst, *errs.values())
    return worst, per_output


class Comm:
    """The library's communicator (NCCL behind the C ABI) plus the second stream the exchange runs on."""

    def __init__(self, torch, dist, b200conv, rank, world, device):
        self.torch, self.b200conv, self.world = torch, b200conv, world
        box = [b200conv.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, device=device)     # the id travels over the host-side rendezvous
        b200conv.comm_init(rank, world, box[0], timeout_ms=120000)
        self.stream = torch.cuda.Stream()
        self.event = torch.cuda.Event()

    def all_reduce_after(self, main, tensor):
        """Sum `tensor` over ranks on the second stream once everything queued on `main` so far has finished."""
        self.event.record(main)
        self.stream.wait_event(self.event)
        self.b200conv.allreduce_sum_f32(tensor.data_ptr(), tensor.numel(), self.stream.cuda_stream)

    def join(self, main):
        main.wait_stream(self.stream)

    def close(self):
        self.b200conv.comm_destroy()


def run_config5(torch, b200conv, dist, comm, rank, world, device, steps, warmup):
    """Config 5: global batch 512, 256 -> 256 channels, 56 x 56, 3x3 pad 1, NCHW; sample i of the global batch comes
    from Generator(5000 + i) (dy: 7000 + i), so every rank count sees the same data.  Per step and rank: forward
    (+bias), dWeight and dBias straight into the fused buffer dW || dB, the all-reduce of that buffer on the second
    stream, dInput under it.  Returns the record for the JSON line."""
    import dp
    import torch.nn.functional as F
    C, HW, GLOBAL = 256, 56, 512
    lo, hi = dp.shard_range(GLOBAL, rank, world)
    n = hi - lo
    hx = dp.seeded_samples((C, HW, HW), 5000, lo, hi)
    hgo = dp.seeded_samples((C, HW, HW), 7000, lo, hi)
    gw = torch.Generator().manual_seed(4999)
    bound = 1.0 / (C * 9) ** 0.5
    hw_ = (torch.rand(C, C, 3, 3, generator=gw) * 2 - 1) * bound
    hb = (torch.rand(C, generator=gw) * 2 - 1) * bound
    x, go, w, b = hx.to(device), hgo.to(device), hw_.to(device), hb.to(device)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    flat, dw, db = dp.fused_gradient_buffer((C, C, 3, 3), True, x)
    p = b200conv.geometry((n, C, HW, HW), C, (3, 3), (1, 1), (1, 1))
    L = b200conv.lib()
    budget = 512 << 20
    ws_bytes = max(max(b200conv.workspace_bytes(p, ph, budget=budget) for ph in (0, 1, 2, 3)), 1)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
    ws2 = torch.empty(ws_bytes, dtype=torch.uint8, device=device)   # dInput runs beside nothing of ours, but keep scratch apart
    main = torch.cuda.current_stream()
    st = main.cuda_stream

    def view(t):
        return b200conv.View4(t.data_ptr(), (ctypes.c_int64 * 4)(*t.stride()))
    xv, wv, gv = view(x), view(w), view(go)

    def step():
        b200conv.check(L.b200_conv2d_forward(ctypes.byref(p), xv, wv, b.data_ptr(), 1, y.data_ptr(), ws.data_ptr(), ws_bytes, 0, st))
        b200conv.check(L.b200_conv2d_dweight(ctypes.byref(p), xv, gv, dw.data_ptr(), ws.data_ptr(), ws_bytes, 0, st))
        b200conv.check(L.b200_conv2d_dbias(ctypes.byref(p), gv, db.data_ptr(), ws.data_ptr(), ws_bytes, st))
        if comm is not None:
            comm.all_reduce_after(main, flat)
        b200conv.check(L.b200_conv2d_dinput(ctypes.byref(p), gv, wv, dx.data_ptr(), ws2.data_ptr(), ws_bytes, 0, st))
        if comm is not None:
            comm.join(main)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = b200conv.launch_count()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    launches = b200conv.launch_count() - launches0
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.cpu())
    # parity of the REDUCED gradients against the single-process oracle on a slice: rows co of dW over input channels ci
    # depend only on dy[:, co] and x[:, ci] of ALL 512 samples, which every rank contributes from its shard
    co = torch.tensor([0, 1, 127, 255], device=device)
    ci = torch.tensor([0, 3, 64, 128, 129, 200, 254, 255], device=device)
    xs, gs = x[:, ci].contiguous(), go[:, co].contiguous()
    if dist is not None:
        xs_all = torch.empty((GLOBAL, *xs.shape[1:]), device=device)
        gs_all = torch.empty((GLOBAL, *gs.shape[1:]), device=device)
        dist.all_gather_into_tensor(xs_all, xs)
        dist.all_gather_into_tensor(gs_all, gs)
        xs, gs = xs_all, gs_all
    record = None
    if rank == 0:
        xs, gs = xs.cpu().double(), gs.cpu().double()
        wdw = torch.ops.aten.convolution_backward(gs, xs, torch.zeros(len(co), len(ci), 3, 3, dtype=torch.float64), None, [1, 1],
                                                  [1, 1], [1, 1], False, [0, 0], 1, [False, True, False])[1]
        errs = {"dw": rel_l2(torch, dw[co][:, ci].cpu(), wdw), "db": rel_l2(torch, db[co].cpu(), gs.sum(dim=(0, 2, 3)))}
        idx = torch.tensor([0, n - 1])
        wy = F.conv2d(hx[idx].double(), hw_.double(), hb.double(), 1, 1)
        wdx = torch.ops.aten.convolution_backward(hgo[idx].double(), hx[idx].double(), hw_.double(), None, [1, 1], [1, 1], [1, 1],
                                                  False, [0, 0], 1, [True, False, False])[0]
        errs["y"] = rel_l2(torch, y[idx.to(device)].cpu(), wy)
        errs["dx"] = rel_l2(torch, dx[idx.to(device)].cpu(), wdx)
        flops = 3 * 2 * GLOBAL * HW * HW * C * C * 9
        record = {"workload": "config 5: global batch 512, 256->256, 56x56, 3x3 pad 1, NCHW, per-sample seeds 5000+i / 7000+i; "
                              "fwd + dWeight + dBias + all-reduce(dW||dB, 2.36 MB, second stream) + dInput",
                  "global_batch": GLOBAL, "per_rank_batch": n, "n_gpus": world, "scaling": "strong", "steps": steps, "warmup": warmup,
                  "ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12, "allreduce_bytes": int(flat.numel()) * 4,
                  "gpu_launches": int(launches), "max_rel_err": max(errs.values()), "rel_err": errs,
                  "parity": "reduced dW rows {0,1,127,255} x input channels {0,3,64,128,129,200,254,255} and dB over all 512 samples, "
                            "y and dX on the first and last image of rank 0, against PyTorch CPU FP64"}
    del x, go, y, dx, ws, ws2
    torch.cuda.empty_cache()
    return record


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="sweep",
                    choices=["sweep", "cfg3", "cfg4", "cfg5", "batch_norm", "group_norm", "attention", "conv3d"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--no-cfg5", action="store_true", help="skip the config-5 record (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--layers", default="", help="comma-separated layer indices (profiling runs)")
    ap.add_argument("--eager", action="store_true",
                    help="launch every kernel of every step from the host instead of replaying one CUDA graph of a step "
                         "(the graph is the default: kernel-to-kernel gaps of 1-2 us instead of 3-9 us)")
    ap.add_argument("--bucket-mb", type=float, default=0.0,
                    help="N > 1: 0 = one exchange of the fused gradient buffer after the last layer (measured fastest: a "
                         "collective CTA and a compute CTA do not fit one SM's register file together, so an all-reduce under "
                         "the persistent kernels delays them by about as much as it hides); > 0 = buckets of consecutive layers "
                         "of at least this many MB, each exchanged under the following layers' kernels")
    ap.add_argument("--reps", type=int, default=10, help="timed repetitions per row of the per-layer workloads")
    ap.add_argument("--shapes", default="", help="shapes of the batch_norm / group_norm / attention workloads")
    ap.add_argument("--graph", action="store_true",
                    help="batch_norm workload: also time `reps` calls inside one CUDA graph (no host launch cost between calls)")
    ap.add_argument("--cpu-baseline", action="store_true",
                    help="batch_norm / group_norm workloads: also time PyTorch's CPU FP32 operator on the host cores")
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
    if args.workload in ("cfg3", "cfg4", "batch_norm", "group_norm", "attention", "conv3d"):
        import bench_workloads
        return getattr(bench_workloads, "run_" + args.workload)(args, torch, b200conv, device, peaks())
    dist, comm = None, None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        # NCCL_DEBUG=VERSION makes NCCL print a banner on stdout, where only the JSON line belongs
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)
        comm = Comm(torch, dist, b200conv, rank, world, device)
    L = b200conv.lib()
    main_stream = torch.cuda.current_stream()
    stream = main_stream.cuda_stream

    if args.workload == "cfg5":
        rec = run_config5(torch, b200conv, dist, comm, rank, world, device, args.steps, args.warmup)
        if rank == 0:
            print(json.dumps(rec))
        if comm is not None:
            comm.close()
            dist.destroy_process_group()
        return

    specs = LAYERS if not args.layers else [LAYERS[int(i)] for i in args.layers.split(",")]
    layers = [Layer(torch, b200conv, spec, cl, hx, hw_, hgo, device)
              for spec, cl, hx, hw_, hgo in host_sweep_tensors(torch, specs, rank, pin=True)]
    ws_bytes = max(max(l.ws_bytes for l in layers), 1)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
    step_flops = sum(l.flops for l in layers)
    # all weight gradients of a step live in one buffer; each layer's slice is exchanged as soon as it is complete
    grad_flat = torch.empty(sum(math.prod(l.w_shape) for l in layers), device=device)
    off = 0
    for l in layers:
        n = math.prod(l.w_shape)
        l.dw = grad_flat[off:off + n].view(l.w_shape)
        off += n
        l.dw_end = off
    pending = [0, 0]          # [start, end) of the gradients computed but not yet exchanged
    BUCKET_FLOATS = int(args.bucket_mb * (1 << 20)) // 4 if args.bucket_mb > 0 else (1 << 62)

    families = {}  # kernel family -> [flops, [event pairs]]
    issue_stream = [stream]   # the stream the library calls are issued on (the capture stream while a graph is recorded)

    def run_layer(l, timed, exchange=True):
        xv, wv, gv = l.views(b200conv)
        calls = (
            ("forward", lambda: L.b200_conv2d_forward(ctypes.byref(l.p), xv, wv, None, 0, l.y.data_ptr(),
                                                      ws.data_ptr(), ws_bytes, 0, issue_stream[0])),
            ("dinput", lambda: L.b200_conv2d_dinput(ctypes.byref(l.p), gv, wv, l.dx.data_ptr(), ws.data_ptr(),
                                                    ws_bytes, 0, issue_stream[0])),
            ("dweight", lambda: L.b200_conv2d_dweight(ctypes.byref(l.p), xv, gv, l.dw.data_ptr(), ws.data_ptr(),
                                                      ws_bytes, 0, issue_stream[0])),
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
        if comm is not None and exchange:
            # the gradients of consecutive layers are adjacent in grad_flat: one exchange after the last layer, or
            # (--bucket-mb) buckets of consecutive layers, each under the kernels of the layers that follow
            pending[1] = l.dw_end
            if pending[1] - pending[0] >= BUCKET_FLOATS or l is layers[-1]:
                comm.all_reduce_after(main_stream, grad_flat[pending[0]:pending[1]])
                pending[0] = pending[1]

    def step(timed=False):
        pending[0] = pending[1] = 0
        for l in layers:
            run_layer(l, timed)
        if comm is not None:
            comm.join(main_stream)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()

    # One step's library calls recorded once into a CUDA graph (same entry points, same kernels, same buffers) and replayed
    # per step: the host then costs one launch per step instead of one per kernel.  The gradient exchange stays outside.
    graph, graph_launches = None, 0      # graph: [(CUDAGraph, end of its layers' gradients in grad_flat)], one per bucket
    if not args.eager and not args.layers:
        # the per-kernel-family times of the roofline object: the same steps with an event pair around every call, BEFORE
        # the timed region, so that the buffers checked afterwards are the ones the timed replays wrote
        for _ in range(args.steps):
            step(timed=True)
        barrier()
        # with --bucket-mb the step is cut where a bucket of gradients is complete: one graph per bucket, its exchange
        # issued behind it on the second stream while the next graph runs
        parts, first = [], 0
        for l in layers:
            if comm is not None and (l.dw_end - first >= BUCKET_FLOATS) and l is not layers[-1]:
                parts.append(l)
                first = l.dw_end
        parts.append(layers[-1])
        try:
            before = b200conv.launch_count()
            graph, it = [], iter(layers)
            for last in parts:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    issue_stream[0] = torch.cuda.current_stream().cuda_stream
                    for l in it:
                        run_layer(l, False, exchange=False)
                        if l is last:
                            break
                graph.append((g, last.dw_end))
            graph_launches = b200conv.launch_count() - before
        except Exception as exc:   # capture not possible here: every kernel is launched from the host, as with --eager
            print(f"bench.py: CUDA graph capture of a step failed ({exc}); running eagerly", file=sys.stderr)
            graph = None
            families.clear()
        issue_stream[0] = stream
        if graph is not None:
            for _ in range(2):
                for g, _end in graph:
                    g.replay()
        barrier()

    def graph_step():
        start = 0
        for g, end in graph:
            g.replay()
            if comm is not None:
                comm.all_reduce_after(main_stream, grad_flat[start:end])
            start = end
        if comm is not None:
            comm.join(main_stream)

    # the sampler starts BEFORE the barrier: opening NVML takes milliseconds, and a rank 0 that entered the timed region
    # late would make every other rank wait for it in the first exchange
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    launches0 = b200conv.launch_count()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    if sampler:
        sampler.mark()
    for _ in range(args.steps):
        if graph is not None:
            graph_step()
        else:
            step(timed=True)
    t_end.record()
    barrier()
    launches = b200conv.launch_count() - launches0 + (graph_launches * args.steps if graph is not None else 0)
    clocks = sampler.stop() if sampler else None
    ms = t_start.elapsed_time(t_end) / args.steps
    status = b200conv.device_status()
    if status != 0:
        raise SystemExit(f"device status word is {status:#x}: a bounded wait gave up; numbers are invalid")

    # ---- the metric's error clause, outside the timed region (outputs of the last timed step) ----
    max_err, err_by_output = (None, None)
    if rank == 0:
        max_err, err_by_output = sampled_max_rel_err(torch, layers, check_dw=(world == 1))

    # ---- end-to-end leg: host buffers in, host buffers out, copies inside the timed region ----
    # Three streams pipeline the step over its layers: uploads of layer i+1, compute of layer i and
    # downloads of layer i-1 overlap (PCIe is full duplex); events order the hand-offs, including the
    # reuse of each layer's device buffers by the next step.
    e2e_ms = float("nan")
    if not args.no_e2e:
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in layers]
        ev_comp = [torch.cuda.Event() for _ in layers]
        ev_out = [torch.cuda.Event() for _ in layers]
        ev_grads = torch.cuda.Event()

        def e2e_step():
            pending[0] = pending[1] = 0
            for i, l in enumerate(layers):
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_comp[i])  # previous step's kernels have finished reading these inputs
                    l.x.copy_(l.hx, non_blocking=True)
                    l.w.copy_(l.hw_, non_blocking=True)
                    l.go.copy_(l.hgo, non_blocking=True)
                    ev_in[i].record(s_in)
                main_stream.wait_event(ev_in[i])
                main_stream.wait_event(ev_out[i])      # previous step's downloads of y/dx/dw have left the buffers
                run_layer(l, False)
                ev_comp[i].record(main_stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[i])
                    l.hy.copy_(l.y, non_blocking=True)
                    l.hdx.copy_(l.dx, non_blocking=True)
                    if comm is None:
                        l.hdw.copy_(l.dw, non_blocking=True)
                    ev_out[i].record(s_out)
            if comm is not None:
                comm.join(main_stream)
                ev_grads.record(main_stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_grads)
                    for i, l in enumerate(layers):
                        l.hdw.copy_(l.dw, non_blocking=True)
                        ev_out[i].record(s_out)

        def e2e_join():
            main_stream.wait_stream(s_in)
            main_stream.wait_stream(s_out)
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

    # ---- CPU baseline beside it (rank 0, N=1): the same sweep on the host cores, median of five steps ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        host = [(l.spec, l.channels_last, l.hx, l.hw_, l.hgo) for l in layers]
        cpu_times, threads = cpu_sweep(torch, host, 5, 2)
        cpu = {"value": step_flops / statistics.median(cpu_times) / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": "the full sweep (12 layer instances, batch 64, both layouts), median of 5 steps after 2 warm-ups, PyTorch CPU "
                         "FP32 conv2d + convolution_backward (the reference's CPU fallback and its tests' ground truth)"}

    h2d_bytes, d2h_bytes = sum(l.h2d for l in layers), sum(l.d2h for l in layers)
    # free the sweep before the sharded configuration takes its 7 GB at N=1
    cfg5 = None
    if not args.no_cfg5 and not args.layers:
        del layers, ws, grad_flat
        torch.cuda.empty_cache()
        cfg5 = run_config5(torch, b200conv, dist, comm, rank, world, device, max(3, min(args.steps, 10)), 3)

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
        traffic = NCU_TRAFFIC_ONE_LAYER.get(dominant, {})
        roofline = {"bound": "tensor", "kernel": dominant, "achieved": ach, "peak": tf32_peak, "unit": "TFLOP/s",
                    "frac": ach / tf32_peak, "frac_of_burst_peak": ach / (pk["bf16"] / 2.0),
                    "frac_of_two_pass_ceiling": ach / (tf32_peak / 2.0),
                    "traffic": traffic.get("bytes_per_launch"), "traffic_layer": traffic.get("layer"),
                    "traffic_note": traffic.get("note"),
                    "peak_source": f"{pk['source']}: sustained bf16 {pk['bf16_sustained']} TFLOP/s / 2 (TF32 rate); the split-precision "
                                   "scheme issues one TF32 and one BF16 pass of equal duration per algorithmic MAC (ceiling = peak/2), "
                                   "three TF32 passes where the dWeight plan keeps 3xTF32 (peak/3)",
                    "families": fam_stats,
                    "families_timed": ("an event pair around every library call in an eager pass of the same steps right before the "
                                       "timed region (the timed region replays a CUDA graph)") if graph is not None
                                      else "an event pair around every library call inside the timed region"}
        line = {
            "metric": "conv2d_fwd_bwd_tflops", "value": world * step_flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": sweep_config(world), "numerics": NUMERICS,
            "max_rel_err": max_err, "max_rel_err_by_output": err_by_output,
            "max_rel_err_sample": "per layer: images 0 and 63 (y, dX), output channels {0, 1, mid, last} over the whole batch (dW"
                                  + ("" if world == 1 else ": skipped at N>1, where dW holds the sum over ranks") + "), PyTorch CPU FP64",
            "clocks": clocks,
            "e2e": {"value": world * step_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": world * h2d_bytes, "d2h_bytes_per_step": world * d2h_bytes, "ms_per_step": e2e_ms,
                    "bytes_are": "whole job (every rank copies its own batch: per rank 1/n_gpus of these)"},
            "gpu_launches": int(launches),
            "launch_mode": (f"{len(graph)} CUDA graph(s) of a step ({graph_launches} kernel launches recorded through the C ABI) replayed per step"
                            if graph is not None else "every kernel launched from the host"),
            "roofline": roofline,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        if cfg5:
            line["config5"] = cfg5
        print(json.dumps(line))
    if comm is not None:
        comm.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
