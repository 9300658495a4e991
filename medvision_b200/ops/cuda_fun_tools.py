"""Forward-only resampling entry points used by the batched CUDA augmentations.

Same signatures as ``affine_2d`` / ``affine_3d`` of medvision/ops/cuda_fun_tools.py:6-91.
"""
import torch

from .. import _C
from ._common import parse_output_size



def _affine(ndim, features, rois, out_size, spatial_scale, sampling_ratio, aligned, order):
    out = parse_output_size(out_size, ndim, name="out_size")
    assert features.dtype in [torch.float32, torch.float16], \
        f'input must be float16 or float32 but got {features.dtype}'
    assert order in [0, 1, 3], f'order {order} is not supported!'
    if order == 0:
        # one sample per output voxel: averaging would blend labels
        sampling_ratio = 1
    assert features.dim() == ndim + 2
    output = features.new_empty((rois.size(0), features.size(1)) + tuple(out))
    # the rois take the dtype (and device) of the image, as rois.type(features.type()) does
    rois = rois.to(device=features.device, dtype=features.dtype)
    fn = _C.affine_2d if ndim == 2 else _C.affine_3d
    fn(features, rois, output, *out, spatial_scale, sampling_ratio, aligned, order)
    return output


def affine_2d(features, rois, out_size, spatial_scale, sampling_ratio=0, aligned=True, order=1):
    """Resample rotated rois of (N, C, H, W) ``features`` to (R, C, out_h, out_w).
    rois: (R, 6) = (batch_index, center_x, center_y, w, h, angle)."""
    return _affine(2, features, rois, out_size, spatial_scale, sampling_ratio, aligned, order)


def affine_3d(features, rois, out_size, spatial_scale, sampling_ratio=0, aligned=True, order=1):
    """Resample rotated rois of (N, C, D, H, W) ``features`` to (R, C, out_d, out_h, out_w).
    rois: (R, 10) = (batch_index, center_x, center_y, center_z, w, h, d, angle_x, angle_y, angle_z)."""
    return _affine(3, features, rois, out_size, spatial_scale, sampling_ratio, aligned, order)


def _apply_offset(ndim, img, offset, order):
    assert img.shape[2:] == offset.shape[2:]
    assert offset.shape[1] == ndim
    assert img.dim() == ndim + 2
    offset = offset.to(img.device)
    if not (img.dtype == torch.float16 and offset.dtype == torch.float32):
        offset = offset.to(img.dtype)  # a float field under a half image is rounded inside the kernel
    output = _C.apply_offset(img.contiguous(), offset.contiguous(), order)
    assert img.shape == output.shape, f"input is {img.shape}, out is {output.shape}"
    return output


def apply_offset_2d(img, offset, order=1):
    """Warp ``img`` (B, C, H, W) by the displacement field ``offset`` (B, 2, H, W) = (dh, dw) in pixels:
    out[b, c, h, w] = interp(img[b, c], (h + dh, w + dw)).  Same signature as
    medvision/ops/cuda_fun_tools.py:94."""
    return _apply_offset(2, img, offset, order)


def apply_offset_3d(img, offset, order=1):
    """3D: ``img`` (B, C, D, H, W), ``offset`` (B, 3, D, H, W) = (dd, dh, dw).  Same signature as
    medvision/ops/cuda_fun_tools.py:133."""
    return _apply_offset(3, img, offset, order)


def _affine_label(ndim, seg, rois, out_size, spatial_scale, aligned):
    assert seg.dim() == ndim + 2 and len(out_size) == ndim
    rois = rois.to(device=seg.device, dtype=torch.float32)
    if seg.dtype in _C._LABEL_DTYPES:
        out = torch.empty((rois.shape[0], seg.shape[1], *out_size), dtype=torch.int32, device=seg.device)
        if _C.affine_label(seg, rois, out, tuple(int(v) for v in out_size), spatial_scale, aligned):
            return out
    fn = affine_2d if ndim == 2 else affine_3d
    return fn(seg.float(), rois, out_size, spatial_scale, 1, aligned, 0).int()


def affine_fields_3d(image, seg, rois, out_size, spatial_scale=1.0, aligned=True, order=1, rois_image=None):
    """An image field and a label field over the same volumes, resampled with the same rois in one go:
    returns ``(affine_3d(image, rois, out_size, spatial_scale, 1, aligned, order),
    affine_label_3d(seg, rois, out_size, spatial_scale, aligned))`` -- what the reference's transforms
    compute with two ``affine_3d`` calls (medvision/aug_cuda_batch/aug_spatial.py:404-493).
    ``rois``: float32 (R, 10); ``rois_image``: the same rois already in the image's dtype, if the caller has them."""
    assert order in [0, 1], f'order {order} is not supported!'
    out = tuple(int(v) for v in out_size)
    rois = rois.to(device=image.device, dtype=torch.float32)
    if rois_image is None:
        rois_image = rois.to(image.dtype)
    if seg.dtype not in _C._LABEL_DTYPES or image.dtype not in (torch.float16, torch.float32) or image.dim() != 5:
        return (affine_3d(image, rois_image, out, spatial_scale, 1, aligned, order),
                affine_label_3d(seg, rois, out, spatial_scale, aligned))
    image_out = image.new_empty((rois.shape[0], image.shape[1]) + out)
    label_out = torch.empty((rois.shape[0], seg.shape[1]) + out, dtype=torch.int32, device=image.device)
    _C.affine_fields_3d(image, rois_image, image_out, seg, rois, label_out, out, spatial_scale, aligned, order)
    return image_out, label_out


def affine_label_2d(seg, rois, out_size, spatial_scale=1.0, aligned=True):
    """Label map (N, C, H, W) of an integer dtype -> int32 (R, C, oh, ow): what the reference's
    augmentations compute as ``affine_2d(seg.float(), rois, out_size, spatial_scale, 1, aligned,
    0).int()`` (medvision/aug_cuda_batch/aug_spatial.py:158-194), in one kernel on the integers."""
    return _affine_label(2, seg, rois, out_size, spatial_scale, aligned)


def affine_label_3d(seg, rois, out_size, spatial_scale=1.0, aligned=True):
    """3D: (N, C, D, H, W) -> int32 (R, C, od, oh, ow)."""
    return _affine_label(3, seg, rois, out_size, spatial_scale, aligned)
