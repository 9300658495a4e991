"""Displacement-field warp (apply_offset_2d / apply_offset_3d; the reference's elastic deformation
runs on it): the CPU restatement against the reference's own deform_2d / deform_3d kernels
(tests/golden/reference_offset_cuda.npz, made by ``tests/golden/make_golden.py offset``) and
against independent formulations; the CUDA kernel, through the C ABI, against the restatement,
the fixtures and -- when the compiled reference kernels are present -- the reference live.

Bars: bit-exact (value-equal; +0 and -0 are not told apart) for half and float, forward only --
the reference's apply_offset has no backward.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import cases  # noqa: E402
from oracle import port, ref  # noqa: E402
from util import FWD_TOL, assert_close, golden_tensor, n_mismatch  # noqa: E402

# fused-multiply-add pattern of the reference build's float kernels (tap sums: bit 3)
REF_FM = 1 | (1 << 1) | (1 << 2) | (1 << 3) | (1 << 5) | (1 << 7) | (1 << 10) | (1 << 13) | \
    (1 << 16) | (1 << 18) | (2 << 20) | (1 << 22)
GOLD_PATH = os.path.join(HERE, "golden", "reference_offset_cuda.npz")
GOLD = np.load(GOLD_PATH) if os.path.exists(GOLD_PATH) else None
CASES = cases.offset_cases()
IDS = [n for n, _ in CASES]


def _fm(dtype):
    return REF_FM if dtype == torch.float32 else 0


# ----------------------------------------------------------------------------- CPU: the restatement
@pytest.mark.parametrize("name,case", CASES, ids=IDS)
def test_restatement_matches_reference_deform_kernels(name, case):
    assert GOLD is not None, "tests/golden/reference_offset_cuda.npz is missing"
    img, off = cases.make_offset_inputs(case)
    want = golden_tensor(GOLD, name, case["dtype"])
    got = port.apply_offset(img, off, case["order"], fma_mode=_fm(case["dtype"]))
    if case["order"] == 3:
        # Catmull-Rom weights: same real numbers, formed as per-axis products instead of the
        # reference's expanded polynomials (equal to ~1e-16 before rounding to the element type)
        assert_close(got, want, FWD_TOL[case["dtype"]], name)
    else:
        assert n_mismatch(got, want) == 0, name


@pytest.mark.parametrize("ndim", [2, 3])
def test_restatement_equals_grid_sample_inside_and_zero_outside(ndim):
    gen = torch.Generator().manual_seed(7)
    spatial = (11, 13) if ndim == 2 else (6, 7, 9)
    img = torch.randn((2, 3) + spatial, generator=gen, dtype=torch.float64)
    off = torch.randn((2, ndim) + spatial, generator=gen, dtype=torch.float64) * 2.0
    got = port.apply_offset(img, off, 1)
    grid = torch.stack(torch.meshgrid(*[torch.arange(n, dtype=torch.float64) for n in spatial], indexing="ij"))[None]
    pos = grid + off
    inside = torch.ones_like(pos[:, 0], dtype=torch.bool)
    for a, n in enumerate(spatial):
        inside &= (pos[:, a] > -1) & (pos[:, a] < n)
    norm = [2 * pos[:, a] / (n - 1) - 1 for a, n in enumerate(spatial)]
    want = F.grid_sample(img, torch.stack(norm[::-1], -1), mode="bilinear", padding_mode="border",
                         align_corners=True)
    assert_close(got, want * inside[:, None], 1e-12)


@pytest.mark.parametrize("order", [0, 1, 3])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_zero_field_is_the_identity_and_whole_voxel_shift_is_a_roll(order, dtype):
    gen = torch.Generator().manual_seed(3)
    img = torch.rand((1, 2, 5, 6, 8), generator=gen).to(dtype)
    zero = torch.zeros((1, 3, 5, 6, 8), dtype=dtype)
    same = port.apply_offset(img, zero, order)
    if order == 3:
        assert_close(same, img, FWD_TOL[dtype])
    else:
        assert torch.equal(same, img)
    shift = zero.clone()
    shift[:, 2] = 3.0  # sample 3 voxels further along w: the image moves left, the tail leaves the image
    got = port.apply_offset(img, shift, order)
    want = torch.zeros_like(img)
    want[..., :5] = img[..., 3:]
    if order == 3:
        assert_close(got, want, FWD_TOL[dtype])
    else:
        assert torch.equal(got, want)


def test_validity_band_is_open_on_both_ends():
    """A sample exactly at -1 or exactly at size is outside (strict comparisons,
    deform_3d_cuda_kernel.cuh:67) -- unlike the roi kernels, whose band [-1, size] is closed;
    just inside of either end it is clamped to the border voxel."""
    img = torch.arange(1.0, 7.0).reshape(1, 1, 1, 6)
    off = torch.zeros(1, 2, 1, 6)
    off[0, 1, 0] = torch.tensor([-1.0, 0.5, 0.0, 2.5, 2.0, 0.999])  # w positions -1, 1.5, 2, 5.5, 6 (= size), 5.999
    got = port.apply_offset(img, off, 1)[0, 0, 0]
    assert got[0] == 0 and got[4] == 0
    assert got[1] == 2.5 and got[2] == 3 and got[3] == 6 and got[5] == 6
    off[0, 0, 0, 2] = -1.0  # h position -1 exactly
    assert port.apply_offset(img, off, 1)[0, 0, 0, 2] == 0


def test_restatement_rejects_bad_arguments():
    img = torch.zeros(1, 1, 4, 4)
    with pytest.raises(ValueError):
        port.apply_offset(img, torch.zeros(1, 2, 4, 4), order=2)


def test_cpu_tensors_are_refused_like_the_reference():
    from medvision_b200.ops import apply_offset_2d, apply_offset_3d
    with pytest.raises(RuntimeError, match="Not implemented on the CPU"):
        apply_offset_2d(torch.zeros(1, 1, 4, 4), torch.zeros(1, 2, 4, 4))
    with pytest.raises(RuntimeError, match="Not implemented on the CPU"):
        apply_offset_3d(torch.zeros(1, 1, 4, 4, 4), torch.zeros(1, 3, 4, 4, 4))
    with pytest.raises(AssertionError):
        apply_offset_3d(torch.zeros(1, 1, 4, 4, 4), torch.zeros(1, 2, 4, 4, 4))


# ----------------------------------------------------------------------------- GPU: the kernel
def _lib_apply(img, off, order):
    from medvision_b200.ops import apply_offset_2d, apply_offset_3d
    fn = apply_offset_2d if img.dim() == 4 else apply_offset_3d
    out = fn(img.cuda(), off.cuda(), order)
    torch.cuda.synchronize()
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("name,case", CASES, ids=IDS)
def test_kernel_bit_exact_against_restatement_fixture_and_live_reference(name, case):
    img, off = cases.make_offset_inputs(case)
    got = _lib_apply(img, off, case["order"])
    want = port.apply_offset(img, off, case["order"], fma_mode=_fm(case["dtype"]))
    if case["order"] == 3 and case["dtype"] == torch.float32:
        # device and host evaluate the double-precision weight products with different contraction
        assert_close(got, want, FWD_TOL[case["dtype"]], name + " vs restatement")
    else:
        assert n_mismatch(got, want) == 0, name + " vs restatement"
    assert GOLD is not None
    gold = golden_tensor(GOLD, name, case["dtype"])
    if case["order"] == 3:
        assert_close(got, gold, FWD_TOL[case["dtype"]], name + " vs fixture")
    else:
        assert n_mismatch(got, gold) == 0, name + " vs fixture"
    if ref.available():
        live = ref.apply_offset(img.cuda(), off.cuda(), case["order"])
        if case["order"] == 3:
            assert_close(got, live, FWD_TOL[case["dtype"]], name + " vs live reference")
        else:
            assert n_mismatch(got, live) == 0, name + " vs live reference"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("spatial", [(1, 1, 1), (3, 1, 5), (4, 5, 2), (1, 7), (6, 1), (2, 2)])
def test_kernel_on_degenerate_and_odd_shapes(dtype, spatial):
    gen = torch.Generator().manual_seed(sum(spatial))
    ndim = len(spatial)
    img = torch.rand((3, 2) + spatial, generator=gen).to(dtype)
    off = (torch.randn((3, ndim) + spatial, generator=gen) * 1.5).to(dtype)
    for order in (0, 1):
        got = _lib_apply(img, off, order)
        assert n_mismatch(got, port.apply_offset(img, off, order, fma_mode=_fm(dtype))) == 0


@pytest.mark.gpu
def test_kernel_with_unaligned_views_and_empty_batch():
    from medvision_b200 import _C
    gen = torch.Generator().manual_seed(11)
    # an offset field whose storage starts one element into an allocation: the vector path must not be taken
    base = torch.randn(2 * 3 * 4 * 6 * 8 + 1, generator=gen).half().cuda()
    off = base[1:].view(2, 3, 4, 6, 8)
    img = torch.rand(2, 2, 4, 6, 8, generator=gen).half().cuda()
    assert off.data_ptr() % 4 == 2
    eye = torch.empty(2, 2, 1, 1, 1, device="meta")
    out = _C.deform_3d(img, eye, torch.empty(2, device="meta"), off, 1, 1, 1, 1, 1, 1, 0, 0, 0, 1, 1, 1, 1, 1, 64, 1)
    torch.cuda.synchronize()
    assert n_mismatch(out, port.apply_offset(img, off, 1)) == 0
    empty = _lib_apply(torch.zeros(0, 2, 4, 4), torch.zeros(0, 2, 4, 4), 1)
    assert empty.shape == (0, 2, 4, 4)
    with pytest.raises(NotImplementedError):
        _C.deform_3d(img, eye, torch.empty(2, device="meta"), off, 3, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 64, 1)
    with pytest.raises(RuntimeError, match="order"):
        _lib_apply(torch.zeros(1, 1, 4, 4), torch.zeros(1, 2, 4, 4), 2)


@pytest.mark.gpu
@pytest.mark.parametrize("spatial", [(6, 10, 12), (5, 7, 9), (14, 18)])
def test_float_field_under_a_half_image_is_rounded_on_load(spatial):
    """apply_offset_* casts the field to the image's dtype first (cuda_fun_tools.py:116-119); the
    kernel does that rounding itself when it is handed a float32 field and a half image."""
    gen = torch.Generator().manual_seed(21)
    ndim = len(spatial)
    img = torch.rand((2, 2) + spatial, generator=gen).half().cuda()
    field = (torch.randn((2, ndim) + spatial, generator=gen) * 2).cuda()
    for order in (0, 1, 3):
        fused = _lib_apply(img, field, order)
        assert torch.equal(fused, _lib_apply(img, field.half(), order))
    assert n_mismatch(_lib_apply(img, field, 1), port.apply_offset(img, field.half(), 1)) == 0
    from medvision_b200 import _C
    with pytest.raises(RuntimeError, match="expected scalar type"):
        _C.apply_offset(img.float(), field.half(), 1)


@pytest.mark.gpu
def test_full_size_volume_properties():
    """128 x 320 x 320 half volume (the elastic-deformation working size of a CT crop):
    zero field = identity, whole-voxel field = shifted copy, and a smooth random field against
    the restatement."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    img = torch.rand((1, 2, 128, 320, 320), generator=gen, device="cuda").half()
    off = torch.zeros((1, 3, 128, 320, 320), device="cuda", dtype=torch.float16)
    assert torch.equal(_lib_apply(img, off, 1), img)
    off[:, 0] = 2.0
    off[:, 1] = -3.0
    got = _lib_apply(img, off, 0)
    want = torch.zeros_like(img)
    want[:, :, :126, 3:, :] = img[:, :, 2:, :317, :]
    assert torch.equal(got, want)
    coarse = torch.randn((1, 3, 8, 12, 12), generator=gen, device="cuda") * 6
    field = F.interpolate(coarse, size=(128, 320, 320), mode="trilinear", align_corners=True).half()
    got = _lib_apply(img, field, 1)
    assert n_mismatch(got, port.apply_offset(img, field, 1)) == 0  # whole volume, all host threads
