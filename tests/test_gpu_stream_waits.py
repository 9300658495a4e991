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
