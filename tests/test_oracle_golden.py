"""The CPU restatement (oracle/) against what the reference itself computes.

Runs without a GPU.  Pins:
  * tests/golden/reference_cuda.npz -- outputs of the reference's OWN CUDA kernels (compiled
    unmodified, run on a B200 by tests/golden/make_golden.py) for the seeded cases of
    tests/golden/cases.py;
  * torchvision's CPU roi_align(aligned=False), which is the same algorithm as the reference's
    2D axis-aligned kernel.
"""
import pytest
import torch

import cases
from oracle import port
from util import BWD_TOL, FWD_TOL, assert_close, golden_tensor, load_golden, n_mismatch

# float contraction pattern of the reference build (see oracle/mvr_oracle.cpp, struct Fm)
REF_FM = 1 | (1 << 1) | (1 << 2) | (1 << 3) | (1 << 5) | (1 << 7) | (1 << 10) | (1 << 13) | \
    (1 << 16) | (1 << 18) | (2 << 20) | (1 << 22)

ALL = cases.all_cases()
CASES = [(n, c) for n, c in ALL if not c.get("affine_only")]
CUBIC = [(n, c) for n, c in ALL if c.get("affine_only")]
GOLD = load_golden()


def _kw(c):
    return dict(spatial_scale=c["spatial_scale"], sampling_ratio=c["sampling_ratio"],
                aligned=c["aligned"], order=c["order"])


@pytest.mark.parametrize("name,case", CASES, ids=[n for n, _ in CASES])
def test_forward_matches_reference_kernels(name, case):
    feat, rois, _ = cases.make_inputs(case)
    fm = REF_FM if case["dtype"] == torch.float32 else 0
    out = port.forward(feat, rois, case["out_size"], case["kind"], fma_mode=fm, **_kw(case))
    ref = golden_tensor(GOLD, name + "/fwd", case["dtype"])
    if case["dtype"] == torch.float16:
        # half: every step is a rounded half operation, host and device agree bit for bit
        assert n_mismatch(out, ref) == 0
    else:
        # float: host sinf/cosf differ from the device's by an ulp for some angles
        assert_close(out, ref, FWD_TOL[torch.float32], name)
        if case["kind"] == cases.KIND_BOX:
            assert n_mismatch(out, ref) == 0  # no trigonometry: exact


@pytest.mark.parametrize("name,case", CASES, ids=[n for n, _ in CASES])
def test_backward_matches_reference_kernels(name, case):
    feat, rois, grad = cases.make_inputs(case)
    fm = REF_FM if case["dtype"] == torch.float32 else 0
    gin = port.backward(grad, rois, feat.shape, case["kind"], fma_mode=fm, **_kw(case))
    ref = golden_tensor(GOLD, name + "/bwd", case["dtype"])
    # the device accumulates with atomics in arbitrary order, in the element type
    assert_close(gin, ref, BWD_TOL[case["dtype"]], name)


@pytest.mark.parametrize("name,case", CUBIC, ids=[n for n, _ in CUBIC])
def test_catmull_rom_forward_matches_reference_kernels(name, case):
    feat, rois, _ = cases.make_inputs(case)
    fm = REF_FM if case["dtype"] == torch.float32 else 0
    out = port.forward(feat, rois, case["out_size"], case["kind"], fma_mode=fm, **_kw(case))
    ref = golden_tensor(GOLD, name + "/fwd", case["dtype"])
    # weights are products of per-axis cubics in double instead of the reference's expanded
    # polynomials in double: the same numbers up to ~1e-16 before the rounding to the element type
    assert_close(out, ref, FWD_TOL[case["dtype"]], name)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("sampling_ratio,scale", [(2, 0.5), (0, 1.0), (3, 0.375)])
def test_box_2d_equals_torchvision(dtype, sampling_ratio, scale):
    torchvision = pytest.importorskip("torchvision")
    g = torch.Generator().manual_seed(5)
    feat = torch.randn(2, 3, 40, 50, generator=g, dtype=dtype)
    R = 24
    b = torch.randint(0, 2, (R, 1), generator=g).to(dtype)
    c = torch.rand(R, 2, generator=g, dtype=dtype) * torch.tensor([50, 40], dtype=dtype)
    s = torch.rand(R, 2, generator=g, dtype=dtype) * 40 + 1
    rois = torch.cat([b, (c - s / 2 - 3) / scale, (c + s / 2 + 3) / scale], 1)
    out = port.forward(feat, rois, (7, 5), port.KIND_BOX, scale, sampling_ratio, True, 1)
    f2 = feat.clone().requires_grad_(True)
    tv = torchvision.ops.roi_align(f2, rois, (7, 5), scale, sampling_ratio, aligned=False)
    if scale in (0.5, 1.0) and sampling_ratio in (0, 2):
        assert torch.equal(out, tv.detach())  # every scaling is exact: no room for contraction differences
    assert_close(out, tv.detach(), 1e-6 if dtype == torch.float32 else 1e-13, 'torchvision forward')
    grad = torch.randn(tv.shape, generator=g, dtype=dtype)
    tv.backward(grad)
    gin = port.backward(grad, rois, feat.shape, port.KIND_BOX, scale, sampling_ratio, True, 1)
    assert_close(gin, f2.grad, 1e-6 if dtype == torch.float32 else 1e-13, "torchvision backward")


@pytest.mark.parametrize("ndim", [2, 3])
@pytest.mark.parametrize("kind", [port.KIND_BOX, port.KIND_ROTATED])
@pytest.mark.parametrize("order", [0, 1])
def test_backward_is_adjoint_of_forward(ndim, kind, order):
    """<forward(f), g> == <f, backward(g)> in double precision: the scatter is the exact
    transpose of the gather (what a finite-difference gradient check would establish)."""
    case = dict(ndim=ndim, kind=kind, dtype=torch.float64, order=order, sampling_ratio=2 if order else 1,
                aligned=True, spatial=(11, 13) if ndim == 2 else (6, 7, 9),
                out_size=(4, 5) if ndim == 2 else (3, 4, 5), seed=77 + ndim + kind, N=2, C=2, R=9,
                spatial_scale=0.8)
    feat, rois, grad = cases.make_inputs(case)
    out = port.forward(feat, rois, case["out_size"], kind, **_kw(case))
    gin = port.backward(grad, rois, feat.shape, kind, **_kw(case))
    lhs = float((out * grad).sum())
    rhs = float((feat * gin).sum())
    assert abs(lhs - rhs) <= 1e-10 * max(1.0, abs(lhs))


def test_identity_roi_reproduces_the_volume():
    """A whole-volume rotated roi with output size = volume size and aligned=True samples every
    voxel centre: the output is the input, bit for bit, in half as well."""
    for dtype in (torch.float16, torch.float32):
        g = torch.Generator().manual_seed(3)
        vol = torch.rand(2, 1, 6, 10, 12, generator=g).to(dtype)
        rois = torch.tensor([[0, 6, 5, 3, 12, 10, 6, 0, 0, 0], [1, 6, 5, 3, 12, 10, 6, 0, 0, 0]], dtype=dtype)
        out = port.forward(vol, rois, (6, 10, 12), port.KIND_ROTATED, 1.0, 1, True, 1)
        assert torch.equal(out, vol)


def test_samples_beyond_one_voxel_outside_contribute_zero_but_count():
    # 1x1 image, roi far larger than it: most sub-samples fall outside the [-1, size] band
    feat = torch.ones(1, 1, 1, 1, dtype=torch.float64)
    rois = torch.tensor([[0, -4.0, -4.0, 4.0, 4.0]], dtype=torch.float64)
    out = port.forward(feat, rois, (1, 1), port.KIND_BOX, 1.0, 4, True, 1)
    # 4x4 samples at -3,-1,1,3: only those at -1 and 1 lie inside the band (clamped to the pixel)
    assert float(out) == pytest.approx(4 / 16)


def test_zero_size_rotated_roi():
    feat = torch.rand(1, 1, 5, 5, dtype=torch.float32)
    rois = torch.tensor([[0, 2.5, 2.5, 0.0, 0.0, 0.3]], dtype=torch.float32)
    # aligned=True does not clamp the size: adaptive grid is 0 samples, the output is 0
    out = port.forward(feat, rois, (2, 2), port.KIND_ROTATED, 1.0, 0, True, 1)
    assert torch.count_nonzero(out) == 0
    # aligned=False forces the size to 1
    out = port.forward(feat, rois, (2, 2), port.KIND_ROTATED, 1.0, 0, False, 1)
    assert torch.count_nonzero(out) == 4


def test_nearest_tie_goes_to_the_lower_index():
    feat = torch.arange(16, dtype=torch.float32).reshape(1, 1, 4, 4)
    # one sample exactly in the middle of pixels (1,1),(1,2),(2,1),(2,2)
    rois = torch.tensor([[0, 2.0, 2.0, 1.0, 1.0, 0.0]], dtype=torch.float32)
    out = port.forward(feat, rois, (1, 1), port.KIND_ROTATED, 1.0, 1, True, 0)
    assert float(out) == 5.0


def test_bad_batch_index_is_reported():
    feat = torch.rand(1, 1, 4, 4)
    rois = torch.tensor([[3, 0, 0, 2, 2]], dtype=torch.float32)
    with pytest.raises(IndexError):
        port.forward(feat, rois, (2, 2), port.KIND_BOX)


def test_empty_roi_list():
    feat = torch.rand(1, 2, 4, 4)
    out = port.forward(feat, torch.zeros(0, 5), (2, 2), port.KIND_BOX)
    assert out.shape == (0, 2, 2, 2)


def test_torch_function_baseline_restatement_matches_the_reference_module():
    """The CPU timing baseline 'torch-function RoIAlign' is a restatement too; its pin is an output
    of the reference's own module (tests/golden/make_torch_function_golden.py)."""
    import numpy as np
    import os
    from oracle.torch_function_path import config1_inputs, roi_align_torch_function
    from util import HERE
    z = np.load(os.path.join(HERE, "golden", "torch_function_c1.npz"))
    feat, rois = config1_inputs(n_rois=16)
    feat.requires_grad_(True)
    out = roi_align_torch_function(feat, rois, (7, 7, 7), 1.0, 1)
    assert torch.equal(out.detach(), torch.from_numpy(z["out"]))
    g = torch.Generator().manual_seed(2)
    out.backward(torch.randn(out.shape, generator=g))
    assert torch.allclose(feat.grad.sum(dim=(2, 3, 4)), torch.from_numpy(z["grad_sum"]), rtol=1e-5, atol=1e-5)
    assert torch.allclose(feat.grad[0, 0, 30:34], torch.from_numpy(z["grad_slab"]), rtol=1e-5, atol=1e-6)
