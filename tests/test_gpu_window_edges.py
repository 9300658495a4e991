"""Wide memory operations at the ends of a tensor.

The backward kernels send a tap row's two x-neighbours as one 16-byte reduction (four floats / eight
halves, zeros in the unused slots): an aligned window around the taps, so at the first and the last
elements of a tensor whose ends are not aligned the window would reach into memory that is not the
tensor's.  The kernels must not use such a window: here the tensors are views into a larger buffer at
odd element offsets and with odd sizes, the buffer around them is filled with -0.0 (a reduction that
adds +0.0 to it would turn it into +0.0), and after the calls (a) the results equal those on freshly
allocated tensors and (b) the surroundings are untouched, bit for bit.  The forward is run on such
views too (no tensor map can be made for them, vector accesses are not aligned): same bits as on an
aligned copy.
"""
import pytest
import torch

from util import BWD_TOL, assert_close, bits

pytestmark = pytest.mark.gpu

PAD = 16  # elements of surroundings on either side


def _embedded(shape, dtype, offset):
    """A contiguous tensor of `shape` that starts `offset` elements into a buffer of -0.0."""
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((n + 2 * PAD,), -0.0, dtype=dtype, device="cuda")
    return buf, buf[offset:offset + n].view(shape)


def _surroundings_untouched(buf, offset, n):
    b = bits(buf)
    neg_zero = bits(torch.full((1,), -0.0, dtype=buf.dtype))[0]
    return bool((b[:offset] == neg_zero).all()) and bool((b[offset + n:] == neg_zero).all())


def _rois(kind, shape, R, seed):
    g = torch.Generator().manual_seed(seed)
    N = shape[0]
    nd = len(shape) - 2
    ext = torch.tensor(list(reversed(shape[2:])), dtype=torch.float32)  # (W, H[, D])
    b = torch.randint(0, N, (R, 1), generator=g).float()
    # centres and sizes that reach over every face of the volume, so that first and last elements are taps
    centre = ext / 2 + (torch.rand(R, nd, generator=g) - 0.5) * ext * 0.3
    size = ext * (0.9 + 0.5 * torch.rand(R, nd, generator=g))
    ang = (torch.rand(R, 1 if nd == 2 else 3, generator=g) - 0.5) * 1.0
    # the first two rois: unrotated, centred, a fifth larger than the volume, one on the first and one on the last
    # sample of the batch -- their outermost samples are clamped onto the first / last element of the tensor
    b[0], b[1] = 0, N - 1
    centre[:2] = ext / 2
    size[:2] = ext * 1.2
    ang[:2] = 0
    if kind == "box":
        return torch.cat([b, centre - size / 2, centre + size / 2], 1)
    return torch.cat([b, centre, size, ang], 1)


CASES = [
    # name,            kind,      feature shape,      output,       ratio
    ("dense3d",        "rotated", (2, 1, 9, 11, 13),  (16, 16, 16), 1),   # streaming backward / gather forward
    ("head3d_box",     "box",     (2, 3, 7, 9, 11),   (3, 4, 5),    2),   # flat kernels
    ("head2d_rotated", "rotated", (2, 3, 1, 17, 19),  (1, 6, 7),    2),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("offset", [1, 3, 5])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_backward_windows_stay_inside_the_gradient_tensor(case, offset, dtype):
    from medvision_b200 import _C
    name, kind, shape, out, ratio = case
    nd = 2 if shape[2] == 1 else 3
    fshape = shape if nd == 3 else (shape[0], shape[1]) + shape[3:]
    osize = out if nd == 3 else out[1:]
    rois = _rois(kind, fshape, 7, 11).to(dtype).cuda()
    g = torch.Generator().manual_seed(12)
    grad = torch.randn((rois.size(0), fshape[1]) + tuple(osize), generator=g).to(dtype).cuda()
    if kind == "box":
        fn = _C.roi_align_2d_backward if nd == 2 else _C.roi_align_3d_backward
        args = (*osize, 1.0, ratio, 1)
    else:
        fn = _C.roi_align_rotated_2d_backward if nd == 2 else _C.roi_align_rotated_3d_backward
        args = (*osize, 1.0, ratio, True, 1)
    want = torch.zeros(fshape, dtype=dtype, device="cuda")
    fn(grad, rois, want, *args)
    buf, got = _embedded(fshape, dtype, offset)
    got.zero_()
    fn(grad, rois, got, *args)
    torch.cuda.synchronize()
    assert float(want.float().abs().max()) > 0
    # first and last elements of the tensor did receive gradient (the windows at the ends were exercised)
    assert float(want.flatten()[:4].float().abs().sum()) > 0 and float(want.flatten()[-4:].float().abs().sum()) > 0
    assert_close(got, want, BWD_TOL[dtype], name)
    assert _surroundings_untouched(buf, offset, got.numel()), "a reduction window reached outside the tensor"


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_forward_reads_the_same_values_at_any_alignment(offset):
    """Half volume at an odd element offset, rois with and without a general rotation: the bits of an aligned copy."""
    from medvision_b200 import _C
    shape = (2, 1, 9, 11, 13)
    g = torch.Generator().manual_seed(21)
    buf, feat = _embedded(shape, torch.float16, offset)
    feat.copy_(torch.randn(shape, generator=g).half())
    rois = _rois("rotated", shape, 5, 22).half().cuda()
    out = (16, 16, 16)
    want = torch.empty((5, 1) + out, dtype=torch.float16, device="cuda")
    got = torch.empty_like(want)
    _C.roi_align_rotated_3d_forward(feat.clone(), rois, want, *out, 1.0, 1, True, 1)
    _C.roi_align_rotated_3d_forward(feat, rois, got, *out, 1.0, 1, True, 1)
    torch.cuda.synchronize()
    assert float(want.float().abs().max()) > 0
    assert bool((bits(got) == bits(want)).all())
