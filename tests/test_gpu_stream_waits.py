"""The plane-streaming forward's hand-shakes, tested without faulting anything:

* its bounded waits: a self-test switch makes every producer leave one plane out, so the consumers'
  wait for it runs out after about a millisecond; the kernel must RETURN, report
  MVR_STATUS_TMA_TIMEOUT, and leave the context usable (the next call is correct);
* the early start of the plane-streaming launch behind the gather launch (programmatic dependent
  launch): whatever follows in the stream, or in another stream behind an event, must see the
  results of BOTH launches.
"""
import math

import pytest
import torch

import cases
from oracle import port
from util import n_mismatch

pytestmark = pytest.mark.gpu


def _case(rot, seed, R=6, spatial=(40, 64, 96), dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    D, H, W = spatial
    feat = torch.rand((2, 1, D, H, W), generator=g).to(dtype)
    ext = torch.tensor([W, H, D], dtype=torch.float32)
    b = torch.randint(0, 2, (R, 1), generator=g).float()
    centre = ext / 2 + (torch.rand(R, 3, generator=g) - 0.5) * ext * 0.3
    size = ext * (0.6 + 0.6 * torch.rand(R, 3, generator=g))
    ang = (torch.rand(R, 3, generator=g) * 2 - 1) * math.pi / 6
    if rot == "z":
        ang[:, :2] = 0
    return feat, torch.cat([b, centre, size, ang], 1).to(dtype)


def test_a_plane_that_never_arrives_ends_in_a_status_bit_not_a_hang():
    from medvision_b200 import _C, _lib
    feat, rois = _case("z", 3)
    out_size = (32, 48, 64)
    want = port.forward(feat, rois, out_size, cases.KIND_ROTATED, 1.0, 1, True, 1, trig=port.device_trig(rois))
    f, r = feat.cuda(), rois.cuda()
    out = torch.empty((rois.size(0), 1) + out_size, dtype=feat.dtype, device="cuda")
    _C.last_status()
    prev = _lib.lib.mvr_selftest_tma_skip_plane(3)
    try:
        assert prev == -1
        _C.affine_3d(f, r, out, *out_size, 1.0, 1, True, 1)
        torch.cuda.synchronize()  # returns: every wait was bounded
    finally:
        _lib.lib.mvr_selftest_tma_skip_plane(-1)
    assert _C.last_status() & _lib.MVR_STATUS_TMA_TIMEOUT
    # the context is intact and the next, normal call is right
    out.fill_(float("nan"))
    _C.affine_3d(f, r, out, *out_size, 1.0, 1, True, 1)
    assert n_mismatch(out, want) == 0
    assert _C.last_status() == 0


@pytest.mark.parametrize("rot", ["xyz", "mixed"])
def test_results_of_both_forward_launches_are_visible_to_what_follows(rot):
    """Every roi under a general rotation: the plane-streaming launch has nothing to do and ends at
    once while the gather launch still runs.  `mixed`: both launches work."""
    from medvision_b200 import _C
    feat, rois = _case("xyz", 7, R=12, spatial=(64, 96, 128))
    if rot == "mixed":
        rois[::2, 7:9] = 0
    out_size = (64, 64, 64)
    want = port.forward(feat, rois, out_size, cases.KIND_ROTATED, 1.0, 1, True, 1, trig=port.device_trig(rois))
    f, r = feat.cuda(), rois.cuda()
    out = torch.full((rois.size(0), 1) + out_size, float("nan"), dtype=feat.dtype, device="cuda")
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    _C.affine_3d(f, r, out, *out_size, 1.0, 1, True, 1)
    same_stream = out.clone()                      # a kernel launched right behind, same stream
    done = torch.cuda.Event()
    done.record()
    with torch.cuda.stream(side):
        side.wait_event(done)
        other_stream = out.clone()                 # another stream, ordered by an event only
    torch.cuda.synchronize()
    assert n_mismatch(same_stream, want) == 0
    assert n_mismatch(other_stream, want) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
def test_chained_head_calls_see_each_others_results(dtype):
    """The detection-head kernels are launched as programmatic dependents (a call's CTAs may become resident while
    the call before it drains) and wait for the complete end of what precedes them before touching memory.  A chain
    in which every call reads what the previous one wrote -- forward into the features of the next forward, then
    backward calls accumulating into one gradient tensor -- gives the bits of the same chain run with a device
    synchronisation after every call."""
    from medvision_b200 import _C
    g = torch.Generator().manual_seed(41)
    N, C, S = 16, 8, 24
    feat0 = torch.rand(N, C, S, S, generator=g).to(dtype).cuda()
    b = torch.arange(N).float().view(-1, 1)
    centre = S / 2 + (torch.rand(N, 2, generator=g) - 0.5) * 4
    size = S * (0.7 + 0.2 * torch.rand(N, 2, generator=g))
    ang = (torch.rand(N, 1, generator=g) - 0.5) * 0.6
    rois = torch.cat([b, centre, size, ang], 1).to(dtype).cuda()       # one roi per sample: output shape == feature shape
    grad = torch.randn(N, C, S, S, generator=g).to(dtype).cuda()

    def chain(sync):
        bufs = [feat0, torch.empty_like(feat0), torch.empty_like(feat0)]
        cur = 0
        for _ in range(8):
            nxt = 1 + (cur % 2) if cur else 1
            _C.roi_align_rotated_2d_forward(bufs[cur], rois, bufs[nxt], S, S, 1.0, 2, True, 1)
            if sync:
                torch.cuda.synchronize()
            cur = nxt
        result = bufs[cur].clone()
        gin = torch.zeros_like(feat0, dtype=torch.float32)
        g32, r32 = grad.float(), rois.float()
        for _ in range(8):  # every call adds the same contributions to the same addresses
            _C.roi_align_rotated_2d_backward(g32, r32, gin, S, S, 1.0, 2, True, 1)
            if sync:
                torch.cuda.synchronize()
        return result, gin

    torch.cuda.synchronize()
    want, gwant = chain(True)
    for _ in range(5):
        got, ggot = chain(False)
        torch.cuda.synchronize()
        assert n_mismatch(got, want) == 0
        # eight equal float contributions per address, in whatever order: equal up to the order of float additions
        assert torch.allclose(ggot, gwant, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rot", ["z", "mixed"])
def test_chained_dense_calls_see_each_others_results(rot):
    """A dense rotated forward is two overlapped launches, and the head kernel behind it is a programmatic
    dependent.  A chain of calls in which each resamples the previous result, followed by a head call on the
    last one, gives the bits of the same chain run with a device synchronisation after every call."""
    from medvision_b200 import _C
    g = torch.Generator().manual_seed(43)
    N, D, H, W = 6, 16, 32, 32
    feat0 = torch.rand(N, 1, D, H, W, generator=g).half().cuda()
    ext = torch.tensor([W, H, D], dtype=torch.float32)
    b = torch.arange(N).float().view(-1, 1)
    centre = ext / 2 + (torch.rand(N, 3, generator=g) - 0.5) * 2
    size = ext * (0.8 + 0.3 * torch.rand(N, 3, generator=g))
    ang = (torch.rand(N, 3, generator=g) - 0.5) * 0.5
    ang[:, :2] = 0
    if rot == "mixed":
        ang[::2, :2] = (torch.rand(N, 2, generator=g)[::2] - 0.5) * 0.5
    rois = torch.cat([b, centre, size, ang], 1).half().cuda()
    head_rois = torch.cat([b, centre - size / 4, centre + size / 4], 1).half().cuda()

    def chain(sync):
        bufs = [feat0, torch.empty_like(feat0), torch.empty_like(feat0)]
        cur = 0
        for _ in range(6):
            nxt = 1 if cur != 1 else 2
            _C.affine_3d(bufs[cur], rois, bufs[nxt], D, H, W, 1.0, 1, True, 1)
            if sync:
                torch.cuda.synchronize()
            cur = nxt
        head = torch.empty((N, 1, 3, 3, 3), dtype=torch.float16, device="cuda")
        _C.roi_align_3d_forward(bufs[cur], head_rois, head, 3, 3, 3, 1.0, 2, 1)
        return bufs[cur].clone(), head

    torch.cuda.synchronize()
    want, hwant = chain(True)
    assert float(want.float().abs().max()) > 0
    for _ in range(5):
        got, hgot = chain(False)
        torch.cuda.synchronize()
        assert n_mismatch(got, want) == 0 and n_mismatch(hgot, hwant) == 0
