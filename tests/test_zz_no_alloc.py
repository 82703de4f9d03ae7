"""The allocation-free dWeight entry point (b200_conv2d_dweight_static).

Hosts that own all device memory through their own pool, or that cannot afford the implicit
synchronisation of cudaMalloc/cudaFree inside their loop, call this variant: its split-K scratch
is a fixed 16 MiB array inside the library instead of caller-provided workspace.  The test calls
it through the C ABI twice in a row, with different geometries, so that the second call runs over
whatever the first left in the shared array, and compares each result with the regular entry
point (b200_conv2d_dweight, CUDA-core split-K); both run the same FP32 FMA arithmetic, so they are held
to 5e-6 relative L2 error against each other and against the FP64 oracle (the suite's contract is 1e-4).
A second test brackets the call with the library's allocator counters and the driver's free-memory figure
to show that the call itself allocates nothing.  The file runs last in the suite, and also passes alone
in a fresh process.
"""
import ctypes

import numpy as np
import pytest

import b200conv
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 5e-6


def _case(xshape, cout, kernel, seed, **kw):
    rng = np.random.default_rng(seed)
    g = oracle.geometry(xshape, cout, kernel, **kw)
    x = rng.standard_normal(g.x_shape, dtype=np.float32)
    go = rng.standard_normal(g.y_shape, dtype=np.float32)
    w = np.zeros(g.w_shape, np.float32)
    return g, x, go, w, kw


def test_static_scratch_dweight_matches_regular_entry_point_twice_in_a_row():
    b200conv.init()
    cases = [
        _case((6, 32, 23, 19), 48, (3, 3), 11, padding=(1, 1)),           # many splits, ragged tiles
        _case((3, 16, 17, 17), 24, (3, 5), 12, stride=(2, 1), padding=(1, 2), groups=2),  # smaller dW, fewer splits
    ]
    for g, x, go, w, kw in cases:
        assert g.n * g.oh * g.ow > 256  # the split-K path (and therefore the static array) is in use
        got = b200conv.conv2d_dweight_static(go, x, w.shape, **kw)
        assert "static scratch" in b200conv.last_kernel()
        _, want, _ = b200conv.conv2d_backward(go, x, w, mask=(False, True, False), algo="tiled",
                                              budget=b200conv.STATIC_SCRATCH_BYTES, **kw)
        assert oracle.rel_l2(got, want) <= GATE
        np.testing.assert_allclose(got, want, rtol=5e-4, atol=5e-4)
        # and both agree with the FP64 oracle
        assert oracle.rel_l2(got, oracle.dweight(g, x, go, f64=True)) <= GATE


def test_static_scratch_call_allocates_no_device_memory():
    """Everything the call needs exists before it: inputs, the result buffer, and (after one warm-up call)
    the resolved address of the static array.  Around the measured call the caching allocator's counters
    (bytes in use, bytes cached, cudaMalloc calls) and the free device memory the driver reports must not move."""
    import torch
    b200conv.init()
    g, x, go, w, kw = _case((6, 32, 23, 19), 48, (3, 3), 21, padding=(1, 1))
    p = b200conv.geometry(x.shape, w.shape[0], w.shape[2:], padding=kw["padding"], wcin=w.shape[1])
    xv, gv = b200conv.DeviceView(x), b200conv.DeviceView(go)
    out = b200conv.DeviceBuffer(4 * w.size)
    L = b200conv.lib()
    b200conv.check(L.b200_conv2d_dweight_static(ctypes.byref(p), xv.view4(), gv.view4(), out.ptr, None))  # set-up call
    b200conv.check(L.b200_device_sync())

    def counters():
        stats = (ctypes.c_uint64 * 4)()
        b200conv.check(L.b200_mem_stats(stats))
        return (stats[0], stats[1], stats[2]), torch.cuda.mem_get_info(0)[0]
    torch.cuda.mem_get_info(0)  # the first query creates torch's context: keep it out of the bracket
    brackets = []
    for _ in range(3):  # the driver's figure may move for reasons outside this process: one clean bracket is the proof
        before = counters()
        b200conv.check(L.b200_conv2d_dweight_static(ctypes.byref(p), xv.view4(), gv.view4(), out.ptr, None))
        b200conv.check(L.b200_device_sync())
        after = counters()
        brackets.append((before, after))
        assert after[0] == before[0], brackets    # the library's own allocator never moves
        if after == before:
            break
    assert brackets[-1][0] == brackets[-1][1], brackets
    assert oracle.rel_l2(out.to_numpy(w.shape), oracle.dweight(g, x, go, f64=True)) <= GATE


def test_static_scratch_rejects_oversized_gradients_with_a_clear_error():
    b200conv.init()
    # dW = 1024*1024*3*3 floats = 36 MiB: two partials cannot fit the 16 MiB array.
    p = b200conv.geometry((1, 1024, 20, 20), 1024, (3, 3), padding=(1, 1))
    dummy = b200conv.DeviceBuffer(16)
    v = b200conv.contiguous_view4(dummy.ptr, (1, 1, 1, 1))
    rc = b200conv.lib().b200_conv2d_dweight_static(ctypes.byref(p), v, v, dummy.ptr, None)
    assert rc == -3
    assert "static workspace" in b200conv.lib().b200_last_error().decode()
