"""A caller records the three convolution phases of a layer through the C ABI into a CUDA graph and replays it.

Every entry point takes the stream it launches on and, handed a workspace, allocates nothing and never synchronises,
so the calls can be issued on a capturing stream as they are.  The test records forward + dInput + dWeight of a
layer (one that the tensor-core kernels take and one that the CUDA-core kernels take), replaces the inputs in place,
replays the graph and compares what the replay wrote with PyTorch CPU FP64 on the new inputs."""
import ctypes

import numpy as np
import pytest

import b200conv
from oracle import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

CASES = [
    # xshape, cout, kernel, stride, padding, groups
    ((4, 128, 28, 28), 128, (3, 3), (1, 1), (1, 1), 1),    # transposed strip forward / dInput, strip dWeight + the pass that sums it
    ((4, 64, 30, 30), 64, (3, 3), (1, 1), (1, 1), 1),      # pixel-on-M strip kernels
    ((2, 96, 20, 20), 48, (1, 1), (2, 2), (0, 0), 1),      # 1x1 strided
    ((2, 12, 17, 19), 20, (3, 2), (1, 2), (1, 0), 2),      # CUDA-core kernels (few channels, groups)
]


def _view(t):
    return b200conv.View4(t.data_ptr(), (ctypes.c_int64 * 4)(*t.stride()))


@pytest.mark.parametrize("xshape,cout,kernel,stride,padding,groups", CASES)
def test_captured_layer_replays_on_new_inputs(xshape, cout, kernel, stride, padding, groups):
    lib = b200conv.lib()
    dev = torch.device("cuda", 0)
    p = b200conv.geometry(xshape, cout, kernel, stride, padding, (1, 1), groups)
    wshape = (cout, xshape[1] // groups) + tuple(kernel)
    yshape = (xshape[0], cout, p.oh, p.ow)
    gen = torch.Generator().manual_seed(sum(xshape) + cout)

    def draw():
        return (torch.randn(xshape, generator=gen), torch.randn(wshape, generator=gen) / float(np.sqrt(np.prod(wshape[1:]))),
                torch.randn(cout, generator=gen), torch.randn(yshape, generator=gen))
    first, second = draw(), draw()
    x, w, b, go = (t.to(dev) for t in first)
    y, dx, dw = torch.empty(yshape, device=dev), torch.empty(xshape, device=dev), torch.empty(wshape, device=dev)
    ws_bytes = max(b200conv.workspace_bytes(p, phase, budget=64 << 20) for phase in (0, 1, 2))
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

    def issue(stream):
        b200conv.check(lib.b200_conv2d_forward(ctypes.byref(p), _view(x), _view(w), ctypes.c_void_p(b.data_ptr()), 1,
                                               ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(ws.data_ptr()), ws_bytes, 0, stream))
        b200conv.check(lib.b200_conv2d_dinput(ctypes.byref(p), _view(go), _view(w), ctypes.c_void_p(dx.data_ptr()),
                                              ctypes.c_void_p(ws.data_ptr()), ws_bytes, 0, stream))
        b200conv.check(lib.b200_conv2d_dweight(ctypes.byref(p), _view(x), _view(go), ctypes.c_void_p(dw.data_ptr()),
                                               ctypes.c_void_p(ws.data_ptr()), ws_bytes, 0, stream))

    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        issue(ctypes.c_void_p(side.cuda_stream))       # a first, ordinary pass (one-time attribute opt-ins happen here)
    side.synchronize()
    before = b200conv.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        issue(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    recorded = b200conv.launch_count() - before
    assert recorded >= 3
    for t, src in zip((x, w, b, go), second):
        t.copy_(src.to(dev))
    y.zero_(); dx.zero_(); dw.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert b200conv.device_status() == 0
    xs, wsrc, bs, gs = (t.numpy() for t in second)
    want = oracle.torch_conv_all(xs, wsrc, bs, gs, stride, padding, (1, 1), groups)
    got = (y.cpu().numpy(), dx.cpu().numpy(), dw.cpu().numpy())
    errs = [oracle.rel_l2(a, e) for a, e in zip(got, want[:3])]
    assert max(errs) <= 1e-4, errs
