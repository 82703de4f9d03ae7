"""Python face of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Two layers, both CPU-only and both independent of the shipped CUDA library:

1. ``liboracle.so`` (``conv_oracle.c``): a C restatement of the reference's
   convolution shader arithmetic (direct, implicit-GEMM K order, split-K
   dWeight + finalize, 128-lane tree reductions, Winograd F(2x2,3x3), strided
   GEMM with the addmm epilogue).  Each C function cites the shader lines it
   follows.
2. ``torch_*`` helpers: PyTorch's CPU convolution in FP64/FP32.  This is the
   ground truth the reference's own tests compare the device result against
   (tests/test_conv_dispatch.py:50-70 promote to float64;
   tests/test_convolution.py:21-40 use float32) and the target of the
   reference's CPU fallback (csrc/ops/mm.cpp:1071-1087).

Parity status: pinned (see tests/test_oracle.py and tests/golden/).
Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class ConvParamsC(ctypes.Structure):
    _fields_ = [(k, ctypes.c_uint32) for k in
                ("n", "cin", "cout", "h", "w", "kh", "kw", "oh", "ow",
                 "sh", "sw", "ph", "pw", "dh", "dw", "groups")]


def build(force: bool = False) -> str:
    """Compile liboracle.so next to its source (gcc + OpenMP)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "conv_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "liboracle.so"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.oracle_weight_split_plan.restype = ctypes.c_uint32
    return _LIB


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _opt(a):
    if a is None:
        return None, None
    return _f(a)


@dataclass
class Geometry:
    """The 16 push constants of the reference's ConvParams (convolution.cpp:45-52)."""
    n: int; cin: int; cout: int; h: int; w: int; kh: int; kw: int; oh: int; ow: int
    sh: int; sw: int; ph: int; pw: int; dh: int; dw: int; groups: int

    def c(self) -> ConvParamsC:
        return ConvParamsC(*(getattr(self, k) for k, _ in ConvParamsC._fields_))

    @property
    def x_shape(self): return (self.n, self.cin, self.h, self.w)
    @property
    def w_shape(self): return (self.cout, self.cin // self.groups, self.kh, self.kw)
    @property
    def y_shape(self): return (self.n, self.cout, self.oh, self.ow)

    def flops(self) -> int:
        """Algorithmic FLOPs of one phase: 2*N*OH*OW*Cout*(Cin/g)*kh*kw."""
        return 2 * self.n * self.oh * self.ow * self.cout * (self.cin // self.groups) * self.kh * self.kw


_GEOMETRY_ERRORS = {
    -1: "invalid shapes or parameters",
    -2: "spatial parameters exceed int32 coordinates",
    -3: "effective kernel exceeds padded input",
    -4: "empty output",
}


def geometry(xshape, cout, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1,
             wcin=None) -> Geometry:
    """Validate and derive OH/OW exactly as convolution_params does."""
    n, cin, h, w = xshape
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)
    (kh, kw), (sh, sw), (ph, pw), (dh, dw) = pair(kernel), pair(stride), pair(padding), pair(dilation)
    if wcin is None:
        wcin = cin // groups if groups > 0 and cin % max(groups, 1) == 0 else -1
    p = ConvParamsC()
    rc = lib().oracle_conv_geometry(ctypes.byref(p), *(ctypes.c_int64(int(v)) for v in
                                    (n, cin, cout, h, w, wcin, kh, kw, sh, sw, ph, pw, dh, dw, groups)))
    if rc != 0:
        raise ValueError(_GEOMETRY_ERRORS[rc])
    return Geometry(*(getattr(p, k) for k, _ in ConvParamsC._fields_))


def pack(base: np.ndarray, offset: int, size, stride) -> np.ndarray:
    size = list(size) + [1] * (4 - len(size)) if len(size) < 4 else list(size)
    base, bp = _f(base.reshape(-1))
    sz = (ctypes.c_int64 * 4)(*size)
    st = (ctypes.c_int64 * 4)(*(list(stride) + [0] * (4 - len(stride))))
    out = np.empty(size, np.float32)
    lib().oracle_pack(bp, ctypes.c_int64(offset), sz, st, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)))
    return out


def _call(name, g: Geometry, ins, out_shape, extra=()):
    keep, ptrs = [], []
    for a in ins:
        arr, ptr = _opt(a)
        keep.append(arr)
        ptrs.append(ptr)
    out = np.zeros(out_shape, np.float32)
    pc = g.c()
    getattr(lib(), name)(ctypes.byref(pc), *ptrs, *extra, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)))
    return out


def forward(g, x, w, b=None, order="direct", f64=False):
    name = {"direct": "oracle_forward_direct", "tiled": "oracle_forward_tiled",
            "depthwise": "oracle_forward_depthwise", "winograd_f2": "oracle_forward_winograd_f2"}[order]
    if f64:
        assert order == "direct"
        name += "_f64"
    return _call(name, g, (x, w, b), g.y_shape)


def dinput(g, go, w, order="direct", f64=False):
    name = {"direct": "oracle_dinput_direct", "tiled": "oracle_dinput_tiled"}[order] + ("_f64" if f64 else "")
    return _call(name, g, (go, w), g.x_shape)


def dweight(g, x, go, order="direct", f64=False, span=None):
    if order == "split":
        total = g.n * g.oh * g.ow
        span = span or 256
        splits = 1 + (total - 1) // span
        count = int(np.prod(g.w_shape))
        scratch = np.zeros(splits * count, np.float32)
        return _call("oracle_dweight_split", g, (x, go), g.w_shape,
                     extra=(ctypes.c_uint32(span), scratch.ctypes.data_as(ctypes.POINTER(ctypes.c_float))))
    name = {"direct": "oracle_dweight_direct", "reduce": "oracle_dweight_reduce"}[order] + ("_f64" if f64 else "")
    return _call(name, g, (x, go), g.w_shape)


def dbias(g, go, order="direct", f64=False):
    name = {"direct": "oracle_dbias_direct", "reduce": "oracle_dbias_reduce"}[order] + ("_f64" if f64 else "")
    return _call(name, g, (go,), (g.cout,))


def weight_split_plan(g, budget=64 << 20, tile_k=16, max_grid_z=65535, max_range=(1 << 32) - 1):
    """(span, count, bytes) of csrc/ops/convolution.cpp:209-233; the two limits
    default to common Vulkan device limits and are inputs, not constants of the path."""
    span, nbytes = ctypes.c_uint32(), ctypes.c_uint64()
    pc = g.c()
    count = lib().oracle_weight_split_plan(ctypes.byref(pc), ctypes.c_uint64(budget), ctypes.c_uint32(tile_k),
                                           ctypes.c_uint64(max_grid_z), ctypes.c_uint64(max_range),
                                           ctypes.byref(span), ctypes.byref(nbytes))
    return span.value, count, nbytes.value


def gemm(a: np.ndarray, b: np.ndarray, bias=None, alpha=1.0, beta=0.0, f64=False):
    """Strided GEMM: a and b may be arbitrary 2-D numpy views of float32 bases."""
    assert a.dtype == np.float32 and b.dtype == np.float32
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    out = np.zeros((M, N), np.float32)
    fp = ctypes.POINTER(ctypes.c_float)
    bias_arr, bias_ptr = _opt(bias)
    fn = lib().oracle_gemm_f64 if f64 else lib().oracle_gemm
    fn(ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K),
       ctypes.cast(a.ctypes.data, fp), ctypes.c_int64(a.strides[0] // 4), ctypes.c_int64(a.strides[1] // 4),
       ctypes.cast(b.ctypes.data, fp), ctypes.c_int64(b.strides[0] // 4), ctypes.c_int64(b.strides[1] // 4),
       bias_ptr, ctypes.c_float(alpha), ctypes.c_float(beta), out.ctypes.data_as(fp))
    return out


# --------------------------------------------------------------------------
# Layer 2: PyTorch CPU (the reference tests' ground truth)
# --------------------------------------------------------------------------

def torch_conv_all(x, w, b, go, stride, padding, dilation, groups, dtype="float64"):
    """y, dx, dw, db from PyTorch's CPU kernels; inputs are float32 arrays/tensors,
    promoted to `dtype` for the computation and returned as float32 numpy."""
    import torch
    import torch.nn.functional as F
    dt = getattr(torch, dtype)
    t = lambda a: None if a is None else torch.as_tensor(np.asarray(a)).to(dt)
    xt, wt, bt, got = t(x), t(w), t(b), t(go)
    y = F.conv2d(xt, wt, bt, stride, padding, dilation, groups)
    dx, dw, db = torch.ops.aten.convolution_backward(
        got, xt, wt, [w.shape[0]], list(stride), list(padding), list(dilation), False, [0, 0], groups,
        [True, True, True])
    return tuple(v.to(torch.float32).numpy() for v in (y, dx, dw, db))


def rel_l2(actual, expected) -> float:
    """The gate metric: ||actual - expected||_2 / ||expected||_2 over one output tensor."""
    a = np.asarray(actual, np.float64).ravel()
    e = np.asarray(expected, np.float64).ravel()
    den = np.linalg.norm(e)
    return float(np.linalg.norm(a - e) / den) if den > 0 else float(np.linalg.norm(a - e))
