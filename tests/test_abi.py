"""Host-only checks of the C-ABI boundary: the library loads, exports every symbol the
header declares, and its host logic (geometry validation, candidate selection, workspace
planning) matches the oracle's restatement of the reference.  No device work is issued."""
import ctypes
import os
import re

import pytest

import b200conv
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200conv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(b200conv.LIB_PATH)
    names = _declared()
    assert len(names) >= 30
    for name in names:
        assert hasattr(handle, name), name


def test_binding_covers_the_header():
    assert sorted(b200conv.SIGNATURES) == _declared()


def test_geometry_matches_oracle_on_reference_cases():
    from golden_cases import conv_cases
    for c in conv_cases():
        p = b200conv.geometry(c["xshape"], c["cout"], c["kernel"], c["stride"], c["padding"], c["dilation"],
                              c["groups"])
        g = oracle.geometry(c["xshape"], c["cout"], c["kernel"], c["stride"], c["padding"], c["dilation"],
                            c["groups"])
        assert (p.oh, p.ow) == (g.oh, g.ow)
        assert p.flops() == g.flops()


def test_geometry_rejections_carry_the_reference_messages():
    with pytest.raises(b200conv.B200Error, match="effective kernel exceeds padded input"):
        b200conv.geometry((1, 2, 2, 2), 3, (3, 3), stride=(2, 2))
    with pytest.raises(b200conv.B200Error, match="int32 coordinates"):
        b200conv.geometry((1, 1, 4, 4), 1, (1, 1), stride=(2 ** 31, 1))
    with pytest.raises(b200conv.B200Error, match="invalid shapes or parameters"):
        b200conv.geometry((1, 6, 4, 4), 4, (1, 1), groups=4)
    with pytest.raises(b200conv.B200Error, match="invalid shapes or parameters"):
        b200conv.geometry((1, 6, 4, 4), 6, (1, 1), groups=2, wcin=6)
    with pytest.raises(b200conv.B200Error, match="indexing overflow"):
        b200conv.geometry((70000, 1, 256, 256), 1, (1, 1))


def test_nd_geometry_shapes_and_rejections():
    """b200_convnd_geometry against the restatement's shape formulas and the reference's messages
    (csrc/ops/convolution_nd.cpp:13-40 of the reference)."""
    from oracle import convnd_oracle
    cases = [((2, 4, 4, 5, 6), (8, 2, 2, 3, 2), (1, 2, 2), (1, 1, 0), (1, 1, 2), (0, 0, 0), False, 2),
             ((2, 4, 4, 5, 6), (4, 4, 2, 3, 2), (1, 2, 2), (1, 1, 0), (1, 1, 2), (0, 1, 1), True, 2),
             ((3, 6, 17), (4, 6, 5), (3,), (2,), (1,), (0,), False, 1),
             ((1, 8, 9, 7), (8, 2, 3, 3), (2, 2), (1, 1), (1, 1), (1, 1), True, 4)]
    for xs, ws, s, pd, d, op, tr, g in cases:
        p, shape = b200conv.convnd_geometry(xs, ws, s, pd, d, op, tr, g)
        assert shape == convnd_oracle.output_shape(xs, ws, s, pd, d, op, tr, g)
        rank = len(xs) - 2
        assert p.rank == rank and list(p.in_)[3 - rank:] == list(xs[2:]) and list(p.in_)[:3 - rank] == [1] * (3 - rank)
    with pytest.raises(b200conv.B200Error, match="invalid groups/input channels"):
        b200conv.convnd_geometry((1, 5, 4, 4, 4), (4, 2, 1, 1, 1), 1, 0, 1, groups=2)
    with pytest.raises(b200conv.B200Error, match="weight/channel/group mismatch"):
        b200conv.convnd_geometry((1, 4, 4, 4, 4), (4, 3, 1, 1, 1), 1, 0, 1, groups=2)
    with pytest.raises(b200conv.B200Error, match="invalid output padding"):
        b200conv.convnd_geometry((1, 4, 4, 4, 4), (4, 4, 1, 1, 1), 1, 0, 1, output_padding=1)
    with pytest.raises(b200conv.B200Error, match="invalid output padding"):
        b200conv.convnd_geometry((1, 4, 4, 4, 4), (4, 4, 2, 2, 2), 2, 0, 1, output_padding=2, transposed=True)
    with pytest.raises(b200conv.B200Error, match="invalid or oversized output shape"):
        b200conv.convnd_geometry((1, 4, 2, 4, 4), (4, 4, 3, 3, 3), 1, 0, 1)
    with pytest.raises(b200conv.B200Error, match="spatial addressing exceeds int32"):
        b200conv.convnd_geometry((1, 4, 4), (4, 4, 3), 2 ** 31, 0, 1)
    with pytest.raises(b200conv.B200Error, match="invalid spatial parameters"):
        b200conv.convnd_geometry((1, 4, 4), (4, 4, 3), 0, 0, 1)


def test_workspace_plan_respects_budget_and_alignment():
    p = b200conv.geometry((64, 256, 56, 56), 256, (3, 3), padding=(1, 1))
    dw_bytes = 256 * 256 * 9 * 4
    for budget in (0, dw_bytes, 3 * dw_bytes, 64 << 20, 1 << 30):
        n = b200conv.workspace_bytes(p, b200conv.PHASE_DWEIGHT, b200conv.ALGO_TILED, budget)
        assert n <= budget and n % dw_bytes == 0
        assert n != dw_bytes  # a single partial is never materialised
    assert b200conv.workspace_bytes(p, b200conv.PHASE_FORWARD, b200conv.ALGO_TILED) == 0
    assert b200conv.workspace_bytes(p, b200conv.PHASE_DINPUT, b200conv.ALGO_DIRECT) == 0


def test_forced_candidates_resolve_or_fail_loudly():
    p = b200conv.geometry((1, 2, 14, 15), 3, (3, 5), stride=(2, 1), padding=(1, 2), dilation=(1, 2))
    assert b200conv.select(p, b200conv.PHASE_FORWARD, b200conv.ALGO_DIRECT) == b200conv.ALGO_DIRECT
    assert b200conv.select(p, b200conv.PHASE_FORWARD, b200conv.ALGO_TILED) == b200conv.ALGO_TILED
    with pytest.raises(b200conv.B200Error, match="incompatible"):
        b200conv.select(p, b200conv.PHASE_FORWARD, b200conv.ALGO_WINOGRAD)
    # tiny geometry: the heuristic stays on the one-thread-per-output kernels (convolution.cpp:463-469)
    assert b200conv.select(p, b200conv.PHASE_FORWARD) == b200conv.ALGO_DIRECT


def test_tcgen05_call_on_a_view_beyond_32_bit_offsets_never_truncates_channels():
    """A view that spans 2^31 elements or more leaves the strip kernel; the gather kernel takes it only
    when the reduction channels come in whole blocks of 32 (it has no ragged-block padding), anything
    else goes to the CUDA-core implicit GEMM.  Host arithmetic only: no tensor is allocated."""
    def strides(c, h, w):
        return (c * h * w, h * w, w, 1)
    small = b200conv.geometry((2, 48, 32, 32), 64, (3, 3), padding=(1, 1))
    assert b200conv.tc_route(small, b200conv.PHASE_FORWARD, strides(48, 32, 32)) == 0
    huge48 = b200conv.geometry((64, 48, 16384, 64), 32, (3, 3), padding=(1, 1))     # 3.2e9 elements, ragged block
    assert b200conv.tc_route(huge48, b200conv.PHASE_FORWARD, strides(48, 16384, 64)) == 2
    huge64 = b200conv.geometry((40, 64, 1024, 1024), 64, (3, 3), padding=(1, 1))    # whole blocks of 32
    assert b200conv.tc_route(huge64, b200conv.PHASE_FORWARD, strides(64, 1024, 1024)) == 1
    # dInput: the reduction runs over the output channels
    dx80 = b200conv.geometry((40, 64, 1024, 1024), 80, (1, 1))
    assert b200conv.tc_route(dx80, b200conv.PHASE_DINPUT, strides(80, 1024, 1024)) == 2
    assert b200conv.tc_route(dx80, b200conv.PHASE_FORWARD, strides(64, 1024, 1024)) == 1   # 1x1 filters stay off the transposed strip kernel
    fwd80 = b200conv.geometry((40, 64, 16384, 64), 80, (3, 3), padding=(1, 1))
    assert b200conv.tc_route(fwd80, b200conv.PHASE_FORWARD, strides(64, 16384, 64)) == 3  # 80 output channels: transposed strip kernel (64-bit offsets)
    # a small tensor inside a huge parent (strides of the parent): still beyond 32-bit offsets
    assert b200conv.tc_route(small, b200conv.PHASE_FORWARD, (2 ** 31, 32 * 32, 32, 1)) == 2


def test_auto_selection_without_workspace_stays_off_the_tcgen05_forward_kernels():
    p = b200conv.geometry((8, 64, 56, 56), 64, (3, 3), padding=(1, 1))
    need = b200conv.workspace_bytes(p, b200conv.PHASE_FORWARD, b200conv.ALGO_TC)
    assert need > 0
    for phase in (b200conv.PHASE_FORWARD, b200conv.PHASE_DINPUT):
        assert b200conv.select(p, phase, b200conv.ALGO_AUTO, budget=need) == b200conv.ALGO_TC
        assert b200conv.select(p, phase, b200conv.ALGO_AUTO, budget=0) == b200conv.ALGO_TILED
        assert b200conv.select(p, phase, b200conv.ALGO_AUTO, budget=need - 1) == b200conv.ALGO_TILED
        assert b200conv.workspace_bytes(p, phase, b200conv.ALGO_AUTO, budget=0) == 0
        # a forced candidate keeps asking for its workspace
        assert b200conv.select(p, phase, b200conv.ALGO_TC, budget=0) == b200conv.ALGO_TC
    # dWeight runs unsplit without scratch
    assert b200conv.select(p, b200conv.PHASE_DWEIGHT, b200conv.ALGO_AUTO, budget=0) == b200conv.ALGO_TC
