"""The allocation-free dWeight entry point (b200_conv2d_dweight_static).

Hosts that own all device memory through their own pool, or that cannot afford the implicit
synchronisation of cudaMalloc/cudaFree inside their loop, call this variant: its split-K scratch
is a fixed 16 MiB array inside the library instead of caller-provided workspace.  The test calls
it through the C ABI twice in a row, with different geometries, so that the second call runs over
whatever the first left in the shared array, and compares each result with the regular entry
point (b200_conv2d_dweight, CUDA-core split-K) under the suite's gate of 1e-4 relative L2 error.
It runs last in the suite, and also passes alone in a fresh process.
"""
import numpy as np
import pytest

import b200conv
from oracle import oracle

pytestmark = pytest.mark.gpu
GATE = 1e-4


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


def test_static_scratch_rejects_oversized_gradients_with_a_clear_error():
    b200conv.init()
    # dW = 1024*1024*3*3 floats = 36 MiB: two partials cannot fit the 16 MiB array.
    p = b200conv.geometry((1, 1024, 20, 20), 1024, (3, 3), padding=(1, 1))
    dummy = b200conv.DeviceBuffer(16)
    v = b200conv.contiguous_view4(dummy.ptr, (1, 1, 1, 1))
    import ctypes
    rc = b200conv.lib().b200_conv2d_dweight_static(ctypes.byref(p), v, v, dummy.ptr, None)
    assert rc == -3
    assert "static workspace" in b200conv.lib().b200_last_error().decode()
