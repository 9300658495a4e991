"""TEST INFRASTRUCTURE -- not product code.

Loader for ``oracle/_ref/mvref_C*.so``: the reference's own CUDA kernels of the resampling
path, compiled unmodified for sm_100a by ``make -C oracle ref`` (which needs the reference
checkout; the built file travels with the repository snapshot, the checkout does not).
Exposes the functions under the names ``medvision._C`` gives them, plus thin wrappers
that allocate the result the way the reference's Python layer does.
"""
import glob
import importlib.util
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_mod = None

KIND_BOX, KIND_ROTATED = 0, 1


def available():
    return bool(glob.glob(os.path.join(_HERE, "_ref", "mvref_C*.so")))


def module():
    global _mod
    if _mod is None:
        paths = glob.glob(os.path.join(_HERE, "_ref", "mvref_C*.so"))
        if not paths:
            raise ImportError("oracle/_ref/mvref_C*.so not built (make -C oracle ref)")
        spec = importlib.util.spec_from_file_location("mvref_C", paths[0])
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod


def forward(features, rois, out_size, kind, spatial_scale=1.0, sampling_ratio=0, aligned=True, order=1,
            affine=False):
    """Reference forward on CUDA tensors (medvision/ops/roi_align_nd.py:36-47,
    roi_align_rotated_nd.py:38-48, cuda_fun_tools.py:34-44): new_zeros output, then the kernel.
    The reference launches on the legacy default stream of the current device."""
    m = module()
    ndim = features.dim() - 2
    out = features.new_zeros((rois.size(0), features.size(1)) + tuple(out_size))
    with torch.cuda.device(features.device):
        torch.cuda.current_stream().synchronize()
        if kind == KIND_BOX:
            fn = m.roi_align_2d_forward if ndim == 2 else m.roi_align_3d_forward
            fn(features, rois, out, *out_size, spatial_scale, sampling_ratio, order)
        elif affine:
            fn = m.affine_2d if ndim == 2 else m.affine_3d
            fn(features, rois, out, *out_size, spatial_scale, sampling_ratio, aligned, order)
        else:
            fn = m.roi_align_rotated_2d_forward if ndim == 2 else m.roi_align_rotated_3d_forward
            fn(features, rois, out, *out_size, spatial_scale, sampling_ratio, aligned, order)
        torch.cuda.synchronize()
    return out


def backward(grad_out, rois, feature_size, kind, spatial_scale=1.0, sampling_ratio=0, aligned=True, order=1):
    m = module()
    ndim = len(feature_size) - 2
    grad_in = rois.new_zeros(tuple(feature_size))
    out_size = tuple(grad_out.shape[2:])
    with torch.cuda.device(grad_out.device):
        torch.cuda.current_stream().synchronize()
        if kind == KIND_BOX:
            fn = m.roi_align_2d_backward if ndim == 2 else m.roi_align_3d_backward
            fn(grad_out.contiguous(), rois, grad_in, *out_size, spatial_scale, sampling_ratio, order)
        else:
            fn = m.roi_align_rotated_2d_backward if ndim == 2 else m.roi_align_rotated_3d_backward
            fn(grad_out.contiguous(), rois, grad_in, *out_size, spatial_scale, sampling_ratio, aligned, order)
        torch.cuda.synchronize()
    return grad_in


def apply_offset(img, offset, order=1):
    """The reference's ``apply_offset_2d/3d`` (medvision/ops/cuda_fun_tools.py:94-167) on CUDA
    tensors: identity weight, zero bias, 1x1(x1) kernel, stride 1, one deformable group."""
    m = module()
    ndim = img.dim() - 2
    assert offset.shape[1] == ndim and img.shape[2:] == offset.shape[2:]
    channels = img.shape[1]
    weight = torch.eye(channels, channels, device=img.device).reshape((channels, channels) + (1,) * ndim)
    bias = torch.zeros(channels, device=img.device)
    offset = offset.to(img.device)
    if img.dtype == torch.float16:
        offset, bias, weight = offset.half(), bias.half(), weight.half()
    ones, zeros = (1,) * ndim, (0,) * ndim
    fn = m.deform_2d if ndim == 2 else m.deform_3d
    with torch.cuda.device(img.device):
        torch.cuda.current_stream().synchronize()
        out = fn(img.contiguous(), weight.contiguous(), bias.contiguous(), offset.contiguous(),
                 *ones, *ones, *zeros, *ones, 1, 1, 64, order)
        torch.cuda.synchronize()
    return out
