"""Parity at the five benchmark configurations, at their stated shapes, on the very tensors
bench.py times (bench_workloads.py): the CUDA library through its C ABI against the reference's own
kernels (oracle/_ref, compiled unmodified for sm_100a) run live on the same GPU.

Forward results must be bit-identical.  Float gradients are held to 1e-4 relative (order of the
atomics differs between two runs of any scatter kernel).  Half gradients: the reference
accumulates in half with atomics and is itself only reproducible to a few half ulps of the running
sum, so the library is held (a) to that spread against the reference's run and (b) tightly, 2e-3,
against the restatement with a wide accumulator, which is the sum both are approximating.

Matches medvision/csrc/cuda_aug/affine_3d_cuda_kernel.cuh:14-120,
medvision/csrc/cuda/roi_align_3d_cuda_kernel.cuh:11-202,
medvision/csrc/cuda/roi_align_rotated_2d_cuda_kernel.cuh:15-196,
medvision/csrc/cuda/roi_align_rotated_3d_cuda_kernel.cuh:15-265.
"""
import pytest
import torch

import bench_workloads as wl
from oracle import port, ref
from util import BWD_TOL, assert_close

pytestmark = pytest.mark.gpu

needs_reference = pytest.mark.skipif(
    not ref.available(),
    reason="oracle/_ref/mvref_C*.so is not built (make -C oracle ref needs the reference checkout): "
           "THE CONFIGURATION PARITY TESTS DID NOT RUN")


def mismatches(a, b):
    """Elements that differ, on the device (+0 == -0; a NaN on both sides is a match)."""
    ne = (a != b) & ~(torch.isnan(a) & torch.isnan(b))
    return int(ne.sum().item())


def lib_forward(w, feat, rois, affine=False):
    from medvision_b200 import _C
    out = torch.full((rois.size(0), feat.size(1)) + tuple(w["out_size"]), float("nan"), dtype=feat.dtype, device="cuda")
    nd = feat.dim() - 2
    if w["kind"] == wl.KIND_BOX:
        fn = _C.roi_align_2d_forward if nd == 2 else _C.roi_align_3d_forward
        fn(feat, rois, out, *w["out_size"], 1.0, w["sampling_ratio"], w["order"])
    elif affine:
        fn = _C.affine_2d if nd == 2 else _C.affine_3d
        fn(feat, rois, out, *w["out_size"], 1.0, w["sampling_ratio"], w["aligned"], w["order"])
    else:
        fn = _C.roi_align_rotated_2d_forward if nd == 2 else _C.roi_align_rotated_3d_forward
        fn(feat, rois, out, *w["out_size"], 1.0, w["sampling_ratio"], w["aligned"], w["order"])
    return out


def lib_backward(w, grad, rois, fshape):
    from medvision_b200 import _C
    gin = torch.zeros(tuple(fshape), dtype=grad.dtype, device="cuda")
    nd = len(fshape) - 2
    if w["kind"] == wl.KIND_BOX:
        fn = _C.roi_align_2d_backward if nd == 2 else _C.roi_align_3d_backward
        fn(grad, rois, gin, *w["out_size"], 1.0, w["sampling_ratio"], w["order"])
    else:
        fn = _C.roi_align_rotated_2d_backward if nd == 2 else _C.roi_align_rotated_3d_backward
        fn(grad, rois, gin, *w["out_size"], 1.0, w["sampling_ratio"], w["aligned"], w["order"])
    return gin


def ref_kw(w):
    return dict(spatial_scale=1.0, sampling_ratio=w["sampling_ratio"], aligned=w["aligned"], order=w["order"])


def upstream(shape, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.empty(shape, device="cuda", dtype=torch.float32).normal_(generator=g).to(dtype)


def check_fwd_bwd(w, affine=False, wide_check=True):
    feat = w["features"].cuda()
    rois = w["rois"].to(feat.dtype).cuda()
    out = lib_forward(w, feat, rois, affine)
    gold = ref.forward(feat, rois, w["out_size"], w["kind"], affine=affine, **ref_kw(w))
    assert out.numel() > 0
    assert mismatches(out, gold) == 0, "forward differs from the reference's kernel"
    grad = upstream(out.shape, feat.dtype, 11)
    del out, gold
    gin = lib_backward(w, grad, rois, feat.shape)
    gref = ref.backward(grad, rois, feat.shape, w["kind"], **ref_kw(w))
    assert_close(gin, gref, BWD_TOL[feat.dtype], w["name"] + ": gradient vs the reference's kernel")
    if feat.dtype == torch.float16 and wide_check:
        trig = port.device_trig(rois.cpu()) if w["kind"] == wl.KIND_ROTATED else None
        wide = port.backward(grad.cpu(), rois.cpu(), feat.shape, w["kind"], trig=trig, wide_acc=True, **ref_kw(w))
        return gin, gref, wide
    return gin, gref, None


@needs_reference
def test_config1_roi_align_3d_head_fwd_bwd():
    """RoIAlign 3D, (2,4,64,64,64) fp32, 128 rois, 7x7x7, sampling_ratio 2."""
    check_fwd_bwd(wl.workload_c1())


@needs_reference
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["float32", "float16"])
def test_config2_roi_align_rotated_2d_head_fwd_bwd(dtype):
    """RoIAlignRotated 2D, (8,3,512,512), 512 rois, 14x14, sampling_ratio 2, float and half."""
    gin, gref, wide = check_fwd_bwd(wl.workload_c2(dtype=dtype))
    if wide is not None:
        # both accumulate in half with atomics here: neither may be further from the wide sum than
        # the other by more than the run-to-run spread
        e_lib = float((gin.double().cpu() - wide.double()).abs().max())
        e_ref = float((gref.double().cpu() - wide.double()).abs().max())
        rms = float(wide.double().pow(2).mean().sqrt())
        assert e_lib <= e_ref + BWD_TOL[torch.float16] * rms, (e_lib, e_ref, rms)


@needs_reference
def test_config3_resize_all_four_volumes():
    """Resize 4 x (1,160,512,512) fp16 -> (128,256,256) through affine_3d, forward."""
    w = wl.workload_c3("cuda")
    feat, rois = w["features"], w["rois"].half().cuda()
    out = lib_forward(w, feat, rois, affine=True)
    gold = ref.forward(feat, rois, w["out_size"], w["kind"], affine=True, **ref_kw(w))
    assert mismatches(out, gold) == 0


@needs_reference
def test_config4_random_affine_three_axes_fwd_bwd():
    """RandomAffine (16,1,128,128,128) fp16, rotation about all three axes, forward + backward."""
    w = wl.workload_c4("cuda")
    gin, gref, wide = check_fwd_bwd(w)
    assert_close(gin, wide, 2e-3, "half gradient vs wide accumulation")


@needs_reference
def test_config4_z_rotation_only_fwd_bwd():
    """The same volumes with the rotation the augmentations use (about z only): the plane-streaming
    forward and the register-accumulating backward."""
    w = wl.workload_c4("cuda", small=True)
    w["rois"][:, 7:9] = 0
    gin, gref, wide = check_fwd_bwd(w)
    assert_close(gin, wide, 2e-3, "half gradient vs wide accumulation")


@needs_reference
def test_config5_crops_full_size_forward():
    """CropRandomWithAffine 8 x (1,256,512,512) fp16 -> (512,1,96,96,96), forward, full size."""
    from medvision_b200 import _C
    w = wl.workload_c5("cuda")
    feat, rois = w["features"], w["rois"].half().cuda()
    _C.last_status()  # clear what earlier tests left in the status word
    out = lib_forward(w, feat, rois, affine=True)
    gold = ref.forward(feat, rois, w["out_size"], w["kind"], affine=True, **ref_kw(w))
    assert out.shape == (512, 1, 96, 96, 96)
    assert mismatches(out, gold) == 0
    # the status word stayed clear (no bounded wait ran out, no bad batch index)
    assert _C.last_status() == 0


def test_the_reference_build_travelled_with_the_repository():
    """Makes an absent oracle/_ref visible as a FAILURE of its own instead of six quiet skips."""
    assert ref.available(), "oracle/_ref/mvref_C*.so missing: configuration parity was not checked"
