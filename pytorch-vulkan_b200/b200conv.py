"""ctypes binding of the C-ABI library (include/b200conv.h).

Used by the tests and the benchmark to reach the CUDA kernels without PyTorch in the
loop.  Every call goes to ``libb200conv.so``; there is no Python or CPU implementation
behind these functions, and a missing library or device raises.

The high-level helpers take numpy arrays (any strided float32 view: the bytes spanned by
the view are uploaded as they are and the kernels consume the view in place through
``b200_view4``), mirroring how the reference's operators accept transposed, sliced,
offset, channels-last and broadcast tensors (csrc/ops/convolution.cpp:641-697).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200conv.so")

PHASE_FORWARD, PHASE_DINPUT, PHASE_DWEIGHT, PHASE_DBIAS = 0, 1, 2, 3
ALGO_AUTO, ALGO_DIRECT, ALGO_TILED, ALGO_TC, ALGO_WINOGRAD = 0, 1, 2, 3, 4
ALGO_NAMES = {"auto": 0, "direct": 1, "tiled": 2, "tc": 3, "winograd": 4}
H2D, D2H, D2D = 1, 2, 3
BN_PLANAR, BN_INTERLEAVED = 0, 1
DEFAULT_WORKSPACE = 64 << 20  # TORCH_VULKAN_CONV_WORKSPACE_MB default, convolution.cpp:239-247


class ConvParams(ctypes.Structure):
    _fields_ = [(k, c_int32) for k in ("n", "cin", "cout", "h", "w", "kh", "kw", "oh", "ow",
                                       "sh", "sw", "ph", "pw", "dh", "dw", "groups")]

    def flops(self):
        return 2 * self.n * self.oh * self.ow * self.cout * (self.cin // self.groups) * self.kh * self.kw


class View4(ctypes.Structure):
    _fields_ = [("ptr", c_void_p), ("stride", c_int64 * 4)]


class ConvNdParams(ctypes.Structure):
    """b200_convnd_params: depth/height/width arrays, lower ranks fill the trailing entries."""
    _fields_ = [("rank", c_int32), ("transposed", c_int32), ("n", c_int64), ("cin", c_int64), ("cout", c_int64),
                ("groups", c_int64)] + [(k, c_int64 * 3) for k in ("in_", "out", "k", "stride", "pad", "dilation")]


class B200Error(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"b200conv error {code}: {text}")
        self.code = code


# name -> (restype, argtypes): the complete list of symbols include/b200conv.h declares.
SIGNATURES = {
    "b200_init": (c_int, [c_int]),
    "b200_last_error": (c_char_p, []),
    "b200_device_name": (c_char_p, []),
    "b200_device_sm_count": (c_int, []),
    "b200_malloc": (c_int, [POINTER(c_void_p), c_size_t, c_void_p]),
    "b200_free": (c_int, [c_void_p, c_void_p]),
    "b200_empty_cache": (c_int, []),
    "b200_mem_stats": (c_int, [POINTER(c_uint64)]),
    "b200_host_alloc": (c_int, [POINTER(c_void_p), c_size_t]),
    "b200_host_free": (c_int, [c_void_p]),
    "b200_memcpy": (c_int, [c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "b200_memset": (c_int, [c_void_p, c_int, c_size_t, c_void_p]),
    "b200_gather_strided": (c_int, [c_void_p, c_void_p, c_int, POINTER(c_int64), POINTER(c_int64), c_int, c_void_p]),
    "b200_scatter_strided": (c_int, [c_void_p, c_void_p, c_int, POINTER(c_int64), POINTER(c_int64), c_int, c_void_p]),
    "b200_scatter_add_strided": (c_int, [c_void_p, c_void_p, c_int, POINTER(c_int64), POINTER(c_int64), c_void_p]),
    "b200_sum_strided": (c_int, [c_void_p, c_void_p, c_int, POINTER(c_int64), POINTER(c_int64), c_void_p, c_void_p]),
    "b200_stream_create": (c_int, [POINTER(c_void_p)]),
    "b200_stream_destroy": (c_int, [c_void_p]),
    "b200_stream_sync": (c_int, [c_void_p]),
    "b200_stream_query": (c_int, [c_void_p]),
    "b200_device_sync": (c_int, []),
    "b200_event_create": (c_int, [POINTER(c_void_p), c_int]),
    "b200_event_destroy": (c_int, [c_void_p]),
    "b200_event_record": (c_int, [c_void_p, c_void_p]),
    "b200_event_sync": (c_int, [c_void_p]),
    "b200_event_query": (c_int, [c_void_p]),
    "b200_stream_wait_event": (c_int, [c_void_p, c_void_p]),
    "b200_event_elapsed_ms": (c_int, [c_void_p, c_void_p, POINTER(c_float)]),
    "b200_conv2d_geometry": (c_int, [POINTER(ConvParams)] + [c_int64] * 15),
    "b200_conv2d_select": (c_int, [POINTER(ConvParams), c_int, c_int, c_size_t]),
    "b200_conv2d_tc_route": (c_int, [POINTER(ConvParams), c_int, View4]),
    "b200_conv2d_workspace": (c_size_t, [POINTER(ConvParams), c_int, c_int, c_size_t]),
    "b200_conv2d_forward": (c_int, [POINTER(ConvParams), View4, View4, c_void_p, c_int64, c_void_p, c_void_p,
                                    c_size_t, c_int, c_void_p]),
    "b200_conv2d_forward_fused": (c_int, [POINTER(ConvParams), View4, View4, c_void_p, c_int64, View4, c_int, c_void_p,
                                          c_int, c_void_p, c_size_t, c_int, c_void_p]),
    "b200_conv2d_dinput": (c_int, [POINTER(ConvParams), View4, View4, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "b200_conv_transpose2d_forward": (c_int, [POINTER(ConvParams), View4, View4, c_void_p, c_int64, c_void_p, c_void_p, c_size_t,
                                              c_int, c_void_p]),
    "b200_conv2d_dweight": (c_int, [POINTER(ConvParams), View4, View4, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "b200_conv2d_dweight_static": (c_int, [POINTER(ConvParams), View4, View4, c_void_p, c_void_p]),
    "b200_conv2d_dbias": (c_int, [POINTER(ConvParams), View4, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200_gemm": (c_int, [c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                          c_void_p, c_float, c_float, c_void_p, c_int, c_void_p]),
    "b200_batch_norm_workspace": (c_size_t, [c_int64, c_int64, c_int64, c_int]),
    "b200_batch_norm_forward": (c_int, [c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
                                        c_void_p, c_int64, c_void_p, c_int64, c_int, c_float, c_float, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200_batch_norm_forward_fused": (c_int, [c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
                                              c_void_p, c_int64, c_void_p, c_int64, c_int, c_float, c_float, c_void_p, c_int,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200_batch_norm_backward": (c_int, [c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                         c_int64, c_void_p, c_int64, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_size_t, c_void_p]),
    "b200_group_norm_workspace": (c_size_t, [c_int64, c_int64, c_int64, c_int64]),
    "b200_group_norm_forward": (c_int, [c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                                        c_void_p, c_void_p, c_void_p]),
    "b200_group_norm_backward": (c_int, [c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200_bmm": (c_int, [c_int64] * 4 + [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                         c_int, c_void_p]),
    "b200_attention_workspace": (c_size_t, [c_int64] * 5 + [c_int]),
    "b200_attention_forward": (c_int, [c_int64] * 5 + [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200_attention_lse_finite": (c_int, [c_void_p, c_int64, c_void_p]),
    "b200_attention_backward": (c_int, [c_int64] * 5 + [c_void_p] * 5 + [c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "b200_convnd_geometry": (c_int, [POINTER(ConvNdParams), c_int, c_int64, c_int64, POINTER(c_int64), c_int64, c_int64]
                             + [POINTER(c_int64)] * 5 + [c_int, c_int64]),
    "b200_convnd_forward": (c_int, [POINTER(ConvNdParams), c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "b200_convnd_backward": (c_int, [POINTER(ConvNdParams)] + [c_void_p] * 7),
    "b200_comm_unique_id": (c_int, [c_void_p]),
    "b200_comm_set_timeout_ms": (c_int, [c_int]),
    "b200_comm_init": (c_int, [c_int, c_int, c_void_p]),
    "b200_comm_rank": (c_int, []),
    "b200_comm_size": (c_int, []),
    "b200_allreduce_sum_f32": (c_int, [c_void_p, c_size_t, c_void_p]),
    "b200_comm_destroy": (c_int, []),
    "b200_device_status": (c_int, [POINTER(c_int), c_int]),
    "b200_launch_count": (c_uint64, []),
    "b200_last_kernel": (c_char_p, []),
}

_lib = None


def lib():
    """Load libb200conv.so and declare every prototype.  Raises if the library is absent:
    build it with ``python pytorch-vulkan_b200/build.py``."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} not found: the CUDA library must be built (no fallback exists)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc):
    if rc < 0:
        raise B200Error(rc, lib().b200_last_error().decode())
    return rc


def init(device=-1):
    check(lib().b200_init(device))


def device_status(clear=False):
    """0 unless a bounded device-side wait gave up (synchronises the device)."""
    v = c_int(0)
    check(lib().b200_device_status(ctypes.byref(v), 1 if clear else 0))
    return v.value


def launch_count():
    return int(lib().b200_launch_count())


def last_kernel():
    return lib().b200_last_kernel().decode()


def comm_unique_id() -> bytes:
    """128 opaque bytes that rank 0 creates and every rank passes to comm_init."""
    buf = ctypes.create_string_buffer(128)
    check(lib().b200_comm_unique_id(buf))
    return buf.raw


def comm_init(rank, nranks, unique_id: bytes, timeout_ms=None):
    if len(unique_id) != 128:
        raise ValueError("the communicator id is 128 bytes")
    if timeout_ms is not None:
        check(lib().b200_comm_set_timeout_ms(int(timeout_ms)))
    check(lib().b200_comm_init(rank, nranks, ctypes.create_string_buffer(unique_id, 128)))


def allreduce_sum_f32(ptr, count, stream=None):
    """In-place sum over ranks of `count` floats at device address `ptr`, asynchronous on `stream`."""
    check(lib().b200_allreduce_sum_f32(ptr, count, stream))


def comm_destroy():
    check(lib().b200_comm_destroy())


class DeviceBuffer:
    """A block from the library's caching allocator."""

    def __init__(self, nbytes, stream=None):
        self.nbytes = int(nbytes)
        self.stream = stream
        p = c_void_p()
        check(lib().b200_malloc(ctypes.byref(p), max(self.nbytes, 1), stream))
        self.ptr = p.value

    def free(self):
        if self.ptr:
            check(lib().b200_free(self.ptr, self.stream))
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def upload(self, host_bytes, stream=None):
        check(lib().b200_memcpy(self.ptr, host_bytes, self.nbytes, H2D, stream))

    def to_numpy(self, shape, dtype=np.float32, stream=None):
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        check(lib().b200_memcpy(out.ctypes.data, self.ptr, out.nbytes, D2H, stream))
        check(lib().b200_stream_sync(stream))
        return out


def geometry(xshape, cout, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, wcin=None):
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)
    n, cin, h, w = xshape
    (kh, kw), (sh, sw), (ph, pw), (dh, dw) = pair(kernel), pair(stride), pair(padding), pair(dilation)
    if wcin is None:
        wcin = cin // groups if groups > 0 else -1
    p = ConvParams()
    check(lib().b200_conv2d_geometry(ctypes.byref(p), n, cin, cout, h, w, wcin, kh, kw, sh, sw, ph, pw, dh, dw, groups))
    return p


def _byte_bounds(a):
    lo = hi = a.ctypes.data
    for dim, st in zip(a.shape, a.strides):
        if dim == 0:
            return a.ctypes.data, a.ctypes.data
        if st > 0:
            hi += (dim - 1) * st
        else:
            lo += (dim - 1) * st
    return lo, hi + a.itemsize


class DeviceView:
    """A float32 numpy view uploaded byte-for-byte; `.view4()` describes it to the kernels."""

    def __init__(self, arr, stream=None):
        arr = np.asarray(arr)
        assert arr.dtype == np.float32
        self.shape = arr.shape
        lo, hi = _byte_bounds(arr)
        self.buf = DeviceBuffer(hi - lo, stream)
        if hi > lo:
            check(lib().b200_memcpy(self.buf.ptr, c_void_p(lo), hi - lo, H2D, stream))
            check(lib().b200_stream_sync(stream))  # the numpy memory may be pageable
        self.ptr = self.buf.ptr + (arr.ctypes.data - lo)
        self.strides = [s // 4 for s in arr.strides]

    def view4(self):
        st = list(self.strides) + [0] * (4 - len(self.strides))
        return View4(self.ptr, (c_int64 * 4)(*st))


def contiguous_view4(ptr, shape):
    st, acc = [], 1
    for d in reversed(shape):
        st.append(acc)
        acc *= d
    return View4(ptr, (c_int64 * 4)(*reversed(st)))


def workspace_bytes(p, phase, algo=ALGO_AUTO, budget=DEFAULT_WORKSPACE):
    return int(lib().b200_conv2d_workspace(ctypes.byref(p), phase, algo, budget))


def select(p, phase, algo=ALGO_AUTO, budget=DEFAULT_WORKSPACE):
    return check(lib().b200_conv2d_select(ctypes.byref(p), phase, algo, budget))


def tc_route(p, phase, strides):
    """0 strip kernel, 1 gather kernel, 2 CUDA-core implicit GEMM, 3 transposed strip kernel for a tcgen05 forward / dInput call on an
    activation view with these element strides (host arithmetic only; no device memory is touched)."""
    return check(lib().b200_conv2d_tc_route(ctypes.byref(p), phase, View4(None, (c_int64 * 4)(*strides))))


def _algo(a):
    return ALGO_NAMES[a] if isinstance(a, str) else int(a)


def conv2d_forward(x, w, b=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, algo="auto",
                   budget=DEFAULT_WORKSPACE):
    """y = conv2d(x, w) + b on the device; numpy in, numpy out (contiguous NCHW)."""
    algo = _algo(algo)
    p = geometry(x.shape, w.shape[0], w.shape[2:], stride, padding, dilation, groups, wcin=w.shape[1])
    xv, wv = DeviceView(x), DeviceView(w)
    bv = DeviceView(b) if b is not None else None
    y = DeviceBuffer(4 * p.n * p.cout * p.oh * p.ow)
    ws_n = workspace_bytes(p, PHASE_FORWARD, algo, budget)
    ws = DeviceBuffer(ws_n) if ws_n else None
    check(lib().b200_conv2d_forward(ctypes.byref(p), xv.view4(), wv.view4(), bv.ptr if bv else None,
                                    bv.strides[0] if bv else 0, y.ptr, ws.ptr if ws else None, ws_n, algo, None))
    return y.to_numpy((p.n, p.cout, p.oh, p.ow))


def conv2d_forward_fused(x, w, b=None, residual=None, relu=False, channels_last=False, stride=(1, 1), padding=(0, 0),
                         dilation=(1, 1), groups=1, algo="auto", budget=DEFAULT_WORKSPACE):
    """act(conv2d(x, w) + b + residual) on the device.  Returns the logical NCHW array; with
    channels_last=True the device wrote it as contiguous [n, oh, ow, cout] and the result is a
    channels-last strided view of that memory."""
    algo = _algo(algo)
    p = geometry(x.shape, w.shape[0], w.shape[2:], stride, padding, dilation, groups, wcin=w.shape[1])
    xv, wv = DeviceView(x), DeviceView(w)
    bv = DeviceView(b) if b is not None else None
    rv = DeviceView(residual) if residual is not None else None
    y = DeviceBuffer(4 * p.n * p.cout * p.oh * p.ow)
    ws_n = workspace_bytes(p, PHASE_FORWARD, algo, budget)
    ws = DeviceBuffer(ws_n) if ws_n else None
    null_view = View4(None, (c_int64 * 4)(0, 0, 0, 0))
    check(lib().b200_conv2d_forward_fused(ctypes.byref(p), xv.view4(), wv.view4(), bv.ptr if bv else None,
                                          bv.strides[0] if bv else 0, rv.view4() if rv else null_view, int(bool(relu)),
                                          y.ptr, int(bool(channels_last)), ws.ptr if ws else None, ws_n, algo, None))
    if channels_last:
        return y.to_numpy((p.n, p.oh, p.ow, p.cout)).transpose(0, 3, 1, 2)
    return y.to_numpy((p.n, p.cout, p.oh, p.ow))


def conv2d_backward(go, x, w, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1,
                    mask=(True, True, True), algo="auto", budget=DEFAULT_WORKSPACE):
    """(dx, dw, db) like aten::convolution_backward with an output mask; None where masked off
    (csrc/ops/convolution.cpp:667-697)."""
    algo = _algo(algo)
    p = geometry(x.shape, w.shape[0], w.shape[2:], stride, padding, dilation, groups, wcin=w.shape[1])
    if tuple(go.shape) != (p.n, p.cout, p.oh, p.ow):
        raise ValueError("convolution backward: output gradient shape mismatch")
    gv = DeviceView(go)
    dx = dw = db = None
    L = lib()
    if mask[0]:
        wv = DeviceView(w)
        out = DeviceBuffer(4 * int(np.prod(x.shape)))
        n = workspace_bytes(p, PHASE_DINPUT, algo, budget)
        ws = DeviceBuffer(n) if n else None
        check(L.b200_conv2d_dinput(ctypes.byref(p), gv.view4(), wv.view4(), out.ptr, ws.ptr if ws else None, n, algo, None))
        dx = out.to_numpy(x.shape)
    if mask[1]:
        xv = DeviceView(x)
        out = DeviceBuffer(4 * int(np.prod(w.shape)))
        n = workspace_bytes(p, PHASE_DWEIGHT, algo, budget)
        ws = DeviceBuffer(n) if n else None
        check(L.b200_conv2d_dweight(ctypes.byref(p), xv.view4(), gv.view4(), out.ptr, ws.ptr if ws else None, n, algo, None))
        dw = out.to_numpy(w.shape)
    if mask[2]:
        out = DeviceBuffer(4 * p.cout)
        n = workspace_bytes(p, PHASE_DBIAS, algo, budget)
        ws = DeviceBuffer(n) if n else None
        check(L.b200_conv2d_dbias(ctypes.byref(p), gv.view4(), out.ptr, ws.ptr if ws else None, n, None))
        db = out.to_numpy((p.cout,))
    return dx, dw, db


STATIC_SCRATCH_BYTES = 16 << 20


def conv2d_dweight_static(go, x, w_shape, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
    """dw through b200_conv2d_dweight_static: the split-K scratch lives inside the library, so the
    call itself allocates nothing (the buffers for x, go and dw below are this helper's own)."""
    init()
    p = geometry(x.shape, w_shape[0], w_shape[2:], stride, padding, dilation, groups, wcin=w_shape[1])
    xv, gv = DeviceView(x), DeviceView(go)
    out = DeviceBuffer(4 * int(np.prod(w_shape)))
    check(lib().b200_conv2d_dweight_static(ctypes.byref(p), xv.view4(), gv.view4(), out.ptr, None))
    return out.to_numpy(tuple(w_shape))


def gemm(a, b, bias=None, alpha=1.0, beta=0.0, algo="auto"):
    """C = alpha*a@b + beta*bias[col] (bias None: plain mm); a and b any 2-D float32 views."""
    M, K = a.shape
    K2, N = b.shape
    if K != K2:
        raise ValueError("matrix shapes cannot be multiplied")
    av, bv = DeviceView(a), DeviceView(b)
    biasv = DeviceView(np.ascontiguousarray(bias, np.float32)) if bias is not None else None
    out = DeviceBuffer(4 * M * N)
    if M * N:
        check(lib().b200_gemm(M, N, K, av.ptr, av.strides[0], av.strides[1], bv.ptr, bv.strides[0], bv.strides[1],
                              biasv.ptr if biasv else None, alpha, beta, out.ptr, _algo(algo), None))
    return out.to_numpy((M, N))


def _bn_pack(a, channels_last):
    """Contiguous device layout of a logical [n, c, *spatial] array: as it is (planar) or with the
    channel axis last (interleaved)."""
    a = np.asarray(a, np.float32)
    return np.ascontiguousarray(np.moveaxis(a, 1, -1)) if channels_last else np.ascontiguousarray(a)


def _bn_unpack(flat, shape, channels_last):
    if not channels_last:
        return flat.reshape(shape)
    moved = (shape[0],) + tuple(shape[2:]) + (shape[1],)
    return np.moveaxis(flat.reshape(moved), -1, 1)


def _bn_dims(shape):
    n, c = int(shape[0]), int(shape[1])
    return n, c, int(np.prod(shape[2:], dtype=np.int64))


def batch_norm_forward(x, weight=None, bias=None, running_mean=None, running_var=None, training=True, momentum=0.1,
                       eps=1e-5, channels_last=False, residual=None, relu=False):
    """aten::native_batch_norm on the device (csrc/ops/batch_norm.cpp:21-83).  x: logical [n, c, ...];
    weight / bias / running_*: channel vectors (any strided float32 view) or None.  Returns
    (y, save_mean, save_inv, running_mean, running_var): save_* are empty in evaluation mode, the
    running statistics are the device's values after the call (None where not given)."""
    n, c, s = _bn_dims(x.shape)
    layout = BN_INTERLEAVED if channels_last else BN_PLANAR
    xv = DeviceView(_bn_pack(x, channels_last))
    vec = [DeviceView(v) if v is not None else None for v in (weight, bias, running_mean, running_var)]
    arg = lambda v: (v.ptr if v else None, v.strides[0] if v else 0)
    y = DeviceBuffer(4 * n * c * s)
    sm, si = DeviceBuffer(4 * c), DeviceBuffer(4 * c)
    ws_n = int(lib().b200_batch_norm_workspace(n, c, s, layout))
    ws = DeviceBuffer(ws_n)
    if residual is None and not relu:
        check(lib().b200_batch_norm_forward(n, c, s, layout, xv.ptr, *arg(vec[0]), *arg(vec[1]), *arg(vec[2]), *arg(vec[3]),
                                            int(bool(training)), momentum, eps, y.ptr, sm.ptr, si.ptr, ws.ptr, ws_n, None))
    else:  # y = relu(batch_norm(x) + residual) in the pass that writes y
        rv = DeviceView(_bn_pack(residual, channels_last)) if residual is not None else None
        check(lib().b200_batch_norm_forward_fused(n, c, s, layout, xv.ptr, *arg(vec[0]), *arg(vec[1]), *arg(vec[2]), *arg(vec[3]),
                                                  int(bool(training)), momentum, eps, rv.ptr if rv else None, int(bool(relu)),
                                                  y.ptr, sm.ptr, si.ptr, ws.ptr, ws_n, None))
    out = _bn_unpack(y.to_numpy((n * c * s,)), x.shape, channels_last)

    def back(view, like):  # the (possibly strided) vector as the device left it
        if view is None:
            return None
        raw = np.empty(view.buf.nbytes // 4, np.float32)
        check(lib().b200_memcpy(raw.ctypes.data, view.buf.ptr, raw.nbytes, D2H, None))
        check(lib().b200_stream_sync(None))
        first = (view.ptr - view.buf.ptr) // 4
        return raw[first::view.strides[0] if view.strides[0] else 1][:c].copy()

    empty = np.empty((0,), np.float32)
    return (out, sm.to_numpy((c,)) if training else empty, si.to_numpy((c,)) if training else empty,
            back(vec[2], running_mean), back(vec[3], running_var))


def batch_norm_backward(grad, x, weight, mean, inv_or_var, training=True, eps=1e-5, mask=(True, True, True),
                        channels_last=False):
    """aten::native_batch_norm_backward on the device (csrc/ops/batch_norm.cpp:84-113): (dx, dw, db),
    None where masked off.  mean / inv_or_var: save_mean / save_inv in training mode, the running
    statistics in evaluation mode."""
    if tuple(grad.shape) != tuple(x.shape):
        raise ValueError("batch norm backward: gradient shape mismatch")
    n, c, s = _bn_dims(x.shape)
    layout = BN_INTERLEAVED if channels_last else BN_PLANAR
    xv, gv = DeviceView(_bn_pack(x, channels_last)), DeviceView(_bn_pack(grad, channels_last))
    wv = DeviceView(weight) if weight is not None else None
    mv, iv = DeviceView(mean), DeviceView(inv_or_var)
    dx = DeviceBuffer(4 * n * c * s) if mask[0] else None
    dw = DeviceBuffer(4 * c) if mask[1] else None
    db = DeviceBuffer(4 * c) if mask[2] else None
    ws_n = int(lib().b200_batch_norm_workspace(n, c, s, layout))
    ws = DeviceBuffer(ws_n)
    check(lib().b200_batch_norm_backward(n, c, s, layout, gv.ptr, xv.ptr, wv.ptr if wv else None, wv.strides[0] if wv else 0,
                                         mv.ptr, mv.strides[0], iv.ptr, iv.strides[0], int(bool(training)), eps,
                                         dx.ptr if dx else None, dw.ptr if dw else None, db.ptr if db else None,
                                         ws.ptr, ws_n, None))
    return (_bn_unpack(dx.to_numpy((n * c * s,)), x.shape, channels_last) if dx else None,
            dw.to_numpy((c,)) if dw else None, db.to_numpy((c,)) if db else None)


def _dense(a):
    return None if a is None else DeviceView(np.ascontiguousarray(a, np.float32))


def group_norm_forward(x, groups, weight=None, bias=None, eps=1e-5):
    """aten::native_group_norm on the device (csrc/ops/group_norm.cpp:76-109): (y, mean [n, groups],
    rstd [n, groups]) for x of logical shape [n, c, ...]."""
    n, c, hw = _bn_dims(x.shape)
    xv, wv, bv = _dense(x), _dense(weight), _dense(bias)
    y, mean, rstd = DeviceBuffer(4 * n * c * hw), DeviceBuffer(4 * n * groups), DeviceBuffer(4 * n * groups)
    check(lib().b200_group_norm_forward(n, c, hw, groups, xv.ptr, wv.ptr if wv else None, bv.ptr if bv else None, eps,
                                        y.ptr, mean.ptr, rstd.ptr, None))
    return y.to_numpy(x.shape), mean.to_numpy((n, groups)), rstd.to_numpy((n, groups))


def group_norm_backward(grad, x, mean, rstd, groups, weight=None, mask=(True, True, True)):
    """aten::native_group_norm_backward on the device (csrc/ops/group_norm.cpp:111-155): (dx, dw, db),
    None where masked off."""
    if tuple(grad.shape) != tuple(x.shape):
        raise ValueError("group norm backward: gradient shape mismatch")
    n, c, hw = _bn_dims(x.shape)
    gv, xv, mv, rv, wv = _dense(grad), _dense(x), _dense(mean), _dense(rstd), _dense(weight)
    dx = DeviceBuffer(4 * n * c * hw) if mask[0] else None
    dw = DeviceBuffer(4 * c) if mask[1] else None
    db = DeviceBuffer(4 * c) if mask[2] else None
    ws_n = int(lib().b200_group_norm_workspace(n, c, hw, groups))
    ws = DeviceBuffer(ws_n)
    check(lib().b200_group_norm_backward(n, c, hw, groups, gv.ptr, xv.ptr, mv.ptr, rv.ptr, wv.ptr if wv else None,
                                         dx.ptr if dx else None, dw.ptr if dw else None, db.ptr if db else None,
                                         ws.ptr, ws_n, None))
    return (dx.to_numpy(x.shape) if dx else None, dw.to_numpy((c,)) if dw else None, db.to_numpy((c,)) if db else None)


def conv_transpose2d_forward(x, w, b=None, stride=(1, 1), padding=(0, 0), output_padding=(0, 0), dilation=(1, 1), groups=1,
                             algo="auto", budget=DEFAULT_WORKSPACE):
    """y = conv_transpose2d(x, w) + b on the device; w is [cin, cout / groups, kh, kw] as in PyTorch."""
    algo = _algo(algo)
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)
    (sh, sw), (ph, pw), (oph, opw), (dh, dw) = pair(stride), pair(padding), pair(output_padding), pair(dilation)
    n, cin, h, wd = x.shape
    kh, kw = w.shape[2:]
    oh = (h - 1) * sh - 2 * ph + dh * (kh - 1) + oph + 1
    ow = (wd - 1) * sw - 2 * pw + dw * (kw - 1) + opw + 1
    # the convolution whose input gradient this is: input [n, cout, oh, ow], output [n, cin, h, wd]
    p = geometry((n, w.shape[1] * groups, oh, ow), cin, (kh, kw), (sh, sw), (ph, pw), (dh, dw), groups, wcin=w.shape[1])
    if (p.oh, p.ow) != (h, wd) or w.shape[0] != cin:
        raise ValueError("transposed convolution: output padding or weight shape does not match the input")
    xv, wv = DeviceView(x), DeviceView(w)
    bv = DeviceView(b) if b is not None else None
    y = DeviceBuffer(4 * p.n * p.cin * p.h * p.w)
    ws_n = workspace_bytes(p, PHASE_DINPUT, algo, budget)
    ws = DeviceBuffer(ws_n) if ws_n else None
    check(lib().b200_conv_transpose2d_forward(ctypes.byref(p), xv.view4(), wv.view4(), bv.ptr if bv else None,
                                              bv.strides[0] if bv else 0, y.ptr, ws.ptr if ws else None, ws_n, algo, None))
    return y.to_numpy((p.n, p.cin, p.h, p.w))


def convnd_geometry(xshape, wshape, stride, padding, dilation, output_padding=None, transposed=False, groups=1):
    """b200_convnd_params for x [n, cin, spatial...] and w ([cout, cin/g, k...] or transposed [cin, cout/g, k...])."""
    rank = len(xshape) - 2
    arr = lambda v: (c_int64 * 3)(*([v] * rank if isinstance(v, int) else list(v)))
    p = ConvNdParams()
    check(lib().b200_convnd_geometry(ctypes.byref(p), rank, xshape[0], xshape[1], arr(list(xshape[2:])), wshape[0], wshape[1],
                                     arr(list(wshape[2:])), arr(stride), arr(padding), arr(dilation),
                                     arr(output_padding if output_padding is not None else 0), int(transposed), groups))
    return p, (p.n, p.cout) + tuple(p.out[3 - rank:])


def _upload_dense(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    buf = DeviceBuffer(a.nbytes)
    if a.nbytes:
        check(lib().b200_memcpy(buf.ptr, a.ctypes.data, a.nbytes, H2D, None))
        check(lib().b200_stream_sync(None))
    return buf


def convnd_forward(x, w, b=None, stride=1, padding=0, dilation=1, output_padding=None, transposed=False, groups=1):
    """Generic 1- to 3-D convolution (float32 or int64) through b200_convnd_forward; operands are packed first."""
    dtype = np.int64 if x.dtype == np.int64 else np.float32
    p, yshape = convnd_geometry(x.shape, w.shape, stride, padding, dilation, output_padding, transposed, groups)
    xb, wb = _upload_dense(x, dtype), _upload_dense(w, dtype)
    bb = _upload_dense(b, dtype) if b is not None else None
    y = DeviceBuffer(int(np.prod(yshape)) * np.dtype(dtype).itemsize)
    check(lib().b200_convnd_forward(ctypes.byref(p), xb.ptr, wb.ptr, bb.ptr if bb else None, y.ptr, int(dtype == np.int64), None))
    return y.to_numpy(yshape, dtype)


def convnd_backward(go, x, w, stride=1, padding=0, dilation=1, output_padding=None, transposed=False, groups=1,
                    mask=(True, True, True)):
    """(dx, dw, db) of the generic convolution through b200_convnd_backward; None where the mask is False."""
    p, yshape = convnd_geometry(x.shape, w.shape, stride, padding, dilation, output_padding, transposed, groups)
    if tuple(go.shape) != tuple(yshape):
        raise ValueError("convolution backward: invalid gradient")
    gb, xb, wb = _upload_dense(go, np.float32), _upload_dense(x, np.float32), _upload_dense(w, np.float32)
    dx = DeviceBuffer(4 * x.size) if mask[0] else None
    dw = DeviceBuffer(4 * w.size) if mask[1] else None
    db = DeviceBuffer(4 * p.cout) if mask[2] else None
    check(lib().b200_convnd_backward(ctypes.byref(p), gb.ptr, xb.ptr, wb.ptr, dx.ptr if dx else None, dw.ptr if dw else None,
                                     db.ptr if db else None, None))
    return (dx.to_numpy(x.shape) if dx else None, dw.to_numpy(w.shape) if dw else None, db.to_numpy((p.cout,)) if db else None)


def bmm(a, b, algo="auto"):
    """C[i] = a[i] @ b[i] on the device; a [batch, M, K] and b [batch, K, N] any float32 views."""
    batch, M, K = a.shape
    batch2, K2, N = b.shape
    if batch != batch2 or K != K2:
        raise ValueError("bmm: expected matching batch dimensions and contraction size")
    av, bv = DeviceView(a), DeviceView(b)
    out = DeviceBuffer(4 * batch * M * N)
    check(lib().b200_bmm(batch, M, N, K, av.ptr, *av.strides, bv.ptr, *bv.strides, out.ptr, _algo(algo), None))
    return out.to_numpy((batch, M, N))


MASK_NONE, MASK_ADDITIVE, MASK_BYTES = 0, 1, 2


def _upload_mask(mask):
    """(buffer or None, mask kind): float32 masks are additive, bool masks hide the keys whose entry is False."""
    if mask is None:
        return None, MASK_NONE
    mask = np.asarray(mask)
    if mask.dtype == np.bool_:
        return _upload_dense(mask.view(np.uint8), np.uint8), MASK_BYTES
    return _upload_dense(mask, np.float32), MASK_ADDITIVE


def _rng_words(rng):
    """(seed, offset) -> the four uint32 words the library takes, or None."""
    if rng is None:
        return None
    seed, offset = (int(v) & ((1 << 64) - 1) for v in rng)
    return (ctypes.c_uint32 * 4)(seed & 0xFFFFFFFF, seed >> 32, offset & 0xFFFFFFFF, offset >> 32)


def attention_forward(q, k, v, mask=None, causal=False, scale=None, dropout=0.0, rng=None):
    """(out, lse) = dropout(softmax(q k^T * scale + mask)) v for q [batch, tq, d], k [batch, tk, d], v [batch, tk, dv];
    rng = (seed, offset) of the Philox stream when 0 < dropout < 1."""
    batch, tq, d = q.shape
    tk, dv = k.shape[1], v.shape[2]
    scale = float(scale) if scale is not None else 1.0 / float(np.sqrt(d))
    qv, kv, vv = _dense(q), _dense(k), _dense(v)
    mv, kind = _upload_mask(mask)
    out, lse = DeviceBuffer(4 * batch * tq * dv), DeviceBuffer(4 * batch * tq)
    ws_n = int(lib().b200_attention_workspace(batch, tq, tk, d, dv, 0))
    ws = DeviceBuffer(ws_n)
    check(lib().b200_attention_forward(batch, tq, tk, d, dv, qv.ptr, kv.ptr, vv.ptr, mv.ptr if mv else None, kind, int(bool(causal)),
                                       scale, float(dropout), _rng_words(rng), out.ptr, lse.ptr, ws.ptr, ws_n, None))
    return out.to_numpy((batch, tq, dv)), lse.to_numpy((batch, tq))


def attention_backward(grad, q, k, v, out, lse, mask=None, causal=False, scale=None, mask_grad=False, dropout=0.0, rng=None):
    """(dq, dk, dv) of attention_forward, plus the gradient of the additive mask when mask_grad is set."""
    batch, tq, d = q.shape
    tk, dv = k.shape[1], v.shape[2]
    scale = float(scale) if scale is not None else 1.0 / float(np.sqrt(d))
    gv, qv, kv, vv, ov, lv = (_dense(a) for a in (grad, q, k, v, out, lse))
    mv, kind = _upload_mask(mask)
    dq, dk, dvb = DeviceBuffer(4 * batch * tq * d), DeviceBuffer(4 * batch * tk * d), DeviceBuffer(4 * batch * tk * dv)
    dm = DeviceBuffer(4 * batch * tq * tk) if mask_grad else None
    ws_n = int(lib().b200_attention_workspace(batch, tq, tk, d, dv, 1))
    ws = DeviceBuffer(ws_n)
    check(lib().b200_attention_backward(batch, tq, tk, d, dv, gv.ptr, qv.ptr, kv.ptr, vv.ptr, mv.ptr if mv else None, kind, ov.ptr,
                                        lv.ptr, int(bool(causal)), scale, float(dropout), _rng_words(rng), dq.ptr, dk.ptr, dvb.ptr,
                                        dm.ptr if dm else None, ws.ptr, ws_n, None))
    grads = dq.to_numpy((batch, tq, d)), dk.to_numpy((batch, tk, d)), dvb.to_numpy((batch, tk, dv))
    return grads + (dm.to_numpy((batch, tq, tk)),) if mask_grad else grads
