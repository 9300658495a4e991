"""Single-sample geometric augmentations on the resampling path.

The transforms of medvision/aug_cuda/aug_spatial.py that end in ``affine_2d/3d`` or
``apply_offset_2d/3d``: CudaResize (:20-153), CudaRandomAffine / Scale / Shift / Rotate (:240-483),
CudaRandomElasticDeformation (:485-708, the cubic-interpolation variant) and
CudaCropRandomWithAffine / CenterWithAffine / FirstDetWithAffine (:967-1228).  Fields are
(C, [D,] H, W) CUDA tensors; every transform builds one roi (xyz order, as the reference) and
resamples the sample as a batch of one.  Parameter draws use numpy's global generator in the
reference's order, and the stored parameter dicts have the reference's keys.

Differences: label fields go through the integer resampler (same values, no float copies); the
roi is built once per call, not once per field; detection boxes (``det_fields``) are not
transformed -- that bookkeeping is numpy code outside the resampling path -- and raise
NotImplementedError instead of being silently left in the old frame.
"""
import math

import numpy as np
import torch

from .base import CudaAugBase
from ..ops.cuda_fun_tools import (affine_2d, affine_3d, affine_label_2d, affine_label_3d, apply_offset_2d,
                                  apply_offset_3d)


def _one_roi(dim, center, shape, shifts, scales, rotate):
    """[0, center - shape * shifts / scales, shape / scales, angles] with the rotation about z in 3D."""
    angles = [rotate] if dim == 2 else [0.0, 0.0, rotate]
    return torch.cat([torch.zeros(1), center - shape * shifts / scales, shape / scales,
                      torch.tensor(angles, dtype=torch.float32)]).unsqueeze(0)


def _resample_sample(result, dim, rois, out_size, sampling_ratio, order):
    """Resamples every image field (order ``order``) and label field (nearest) of one sample."""
    out_size = tuple(int(v) for v in out_size)
    fn, label_fn = (affine_2d, affine_label_2d) if dim == 2 else (affine_3d, affine_label_3d)
    for key in result.get('img_fields', []):
        image = result[key]
        assert image.is_cuda, 'image should be cuda'
        assert image.ndim == dim + 1, 'image should be channel, **dim'
        img = fn(image.unsqueeze(0), rois.to(image.device), out_size, 1.0, sampling_ratio, True, order).squeeze(0)
        result[key] = img
        if key == 'img':
            result['img_shape'] = tuple(img.shape)
    for key in result.get('seg_fields', []):
        seg = result[key]
        assert seg.is_cuda, 'seg should be cuda'
        assert seg.ndim == dim + 1, 'seg should be channel, **dim'
        result[key] = label_fn(seg.unsqueeze(0), rois.to(seg.device), out_size, 1.0, True).squeeze(0)
    for _ in result.get('det_fields', []):
        raise NotImplementedError('detection boxes are not transformed by this implementation')


class CudaResize(CudaAugBase):
    def __init__(self, spacing=None, scale=None, factor=None, order=1):
        super().__init__()
        self.always = True
        self.spacing = spacing
        self.scale = scale
        self.factor = factor
        self.order = order
        assert sum([spacing is not None, scale is not None, factor is not None]) == 1

    def __repr__(self):
        return self.__class__.__name__ + '(spacing={}, scale={}, factor={})'.format(self.spacing, self.scale, self.factor)

    @property
    def canBackward(self):
        return True

    def _forward_params(self, result):
        self._init_params(result)
        if self.spacing is not None:
            assert len(self.spacing) == self.dim, f"not match with a {result['img_dim']}D image"
            img_spacing = np.array(result['img_spacing'])
            new_spacing = np.array(self.spacing)
            new_spacing = np.where(new_spacing == -1, img_spacing, new_spacing)
            scale_factor = tuple(img_spacing / new_spacing)
        elif self.scale is not None:
            assert len(self.scale) == self.dim, f"not match with a {result['img_dim']}D image"
            new_shape = np.array(self.scale)
            new_shape = np.where(new_shape == -1, self.image_shape, new_shape)
            scale_factor = tuple(new_shape / self.image_shape)
        else:
            assert len(self.factor) == self.dim, f"not match with a {result['img_dim']}D image"
            scale_factor = tuple(self.factor)
        self.params = scale_factor
        result[self.key_name] = self.params

    def _backward_params(self, result):
        self._init_params(result)
        params = result.pop(self.key_name, None)
        if params:
            self.params = tuple(1 / np.array(params))

    def _rois(self):
        center = torch.tensor([i / 2 for i in self.image_shape[::-1]], dtype=torch.float32)  # dhw => xyz
        shape = torch.tensor(list(self.image_shape[::-1]), dtype=torch.float32)
        return _one_roi(self.dim, center, shape, torch.zeros(self.dim), torch.ones(self.dim), 0.0)

    def apply_to_img(self, result):
        if all(i == 1.0 for i in self.params):
            return
        out_size = tuple(int(i * p) for i, p in zip(self.image_shape, self.params))
        had_spacing = 'img' in result.get('img_fields', []) and 'img_spacing' in result
        _resample_sample(result, self.dim, self._rois(), out_size, 1, self.order)
        if had_spacing:
            result['img_spacing'] = tuple(np.array(result['img_spacing']) / np.array(self.params))

    def apply_to_seg(self, result):
        pass  # done together with the images


class CudaRandomAffine(CudaAugBase):
    def __init__(self, p, scale, shift, rotate, sampling_ratio=1, order=1):
        super().__init__()
        self.p = p
        self.scale = scale
        self.shift = shift
        self.rotate = rotate  # degrees, in the xy plane
        self.sampling_ratio = sampling_ratio
        self.order = order

    def __repr__(self):
        return self.__class__.__name__ + '(dim={}, scale={}, shift={}, rotate={})'.format(
            self.dim, self.scale, self.shift, self.rotate)

    def _draw(self):
        scales = [self.get_range(self.scale, 1), ] * self.dim
        shifts = [self.get_range(self.shift, 0) for _ in range(self.dim)]
        rotate = [math.pi * self.get_range(self.rotate, 0) / 180]
        return scales, shifts, rotate

    def _forward_params(self, result):
        self._init_params(result)
        scales, shifts, rotate = self._draw()
        self.params = {"_scales": scales, "_shifts": shifts, "_rotate": rotate}
        result[self.key_name] = self.params

    def _backward_params(self, result):
        self._init_params(result)
        params = result.get(self.key_name, None)
        if params:
            self.params = {"_scales": list(1 / np.asarray(params["_scales"])),
                           "_shifts": list(-np.asarray(params["_shifts"])),
                           "_rotate": list(-np.asarray(params["_rotate"]))}

    def _rois(self):
        center = torch.tensor([i / 2 for i in self.image_shape[::-1]], dtype=torch.float32)
        shape = torch.tensor(list(self.image_shape[::-1]), dtype=torch.float32)
        return _one_roi(self.dim, center, shape, torch.FloatTensor(self.params["_shifts"]),
                        torch.FloatTensor(self.params["_scales"]), float(self.params["_rotate"][0]))

    def apply_to_img(self, result):
        _resample_sample(result, self.dim, self._rois(), self.image_shape, self.sampling_ratio, self.order)

    def apply_to_seg(self, result):
        pass  # done together with the images


class CudaRandomScale(CudaRandomAffine):
    def __init__(self, p, scale, sampling_ratio=1):
        super().__init__(p, scale=scale, shift=0, rotate=0, sampling_ratio=sampling_ratio)


class CudaRandomShift(CudaRandomAffine):
    def __init__(self, p, shift, sampling_ratio=1):
        super().__init__(p, scale=0, shift=shift, rotate=0, sampling_ratio=sampling_ratio)


class CudaRandomRotate(CudaRandomAffine):
    def __init__(self, p, rotate, sampling_ratio=1):
        super().__init__(p, scale=0, shift=0, rotate=rotate, sampling_ratio=sampling_ratio)


class CudaRandomElasticDeformation(CudaAugBase):
    """Random smooth warp: a coarse grid of random displacements (two outermost control points of
    every axis locked) is blown up to a dense field by one Catmull-Rom ``affine_*`` resample and
    applied with ``apply_offset_*`` -- linear for images, nearest for labels."""

    def __init__(self, p, num_control_points=8, max_displacement: float = 0.8):
        super().__init__()
        self.p = p
        self.num_control_points = num_control_points  # d, h, w order
        self.max_displacement = max_displacement
        self.SPLINE_ORDER = 3
        self.num_locked_borders = 2
        assert max_displacement <= 1.0
        self.tmp_params = None

    def __repr__(self):
        return self.__class__.__name__ + "(p={}, num_control_points={}, max_displacement={})".format(
            self.p, self.num_control_points, self.max_displacement)

    @property
    def canBackward(self):
        return True

    def _forward_params(self, result):
        self.tmp_params = None
        self._init_params(result)
        grid_shape = self.to_tuple(self.num_control_points, self.dim)
        reach = self.max_displacement * (np.array(self.image_shape) / (np.array(grid_shape) - 1)) / 2
        coarse = 2 * np.random.rand(*grid_shape, self.dim).astype(np.float32) - 1  # [-1, 1)
        coarse *= reach.astype(np.float32)
        for axis in range(self.dim):
            locked = [slice(None)] * self.dim
            for i in range(self.num_locked_borders):
                for pos in (i, -1 - i):
                    locked[axis] = pos
                    coarse[tuple(locked)] = 0
        self.params = coarse
        result[self.key_name] = self.params

    def _backward_params(self, result):
        self.tmp_params = None
        self._init_params(result)
        params = result.pop(self.key_name, None)
        if params is not None:
            self.params = -params

    def dense_field(self, device):
        """(dim, *image_shape) float32 displacement field on ``device``."""
        if self.tmp_params is None:
            coarse = torch.from_numpy(self.params).permute(self.dim, *range(self.dim)) / 2  # halved to smooth
            grid = coarse.shape[1:]
            center = torch.tensor([i / 2 for i in grid[::-1]], dtype=torch.float32)
            shape = torch.tensor(list(grid[::-1]), dtype=torch.float32) - (2 * self.num_locked_borders - 1)
            rois = _one_roi(self.dim, center, shape, torch.zeros(self.dim), torch.ones(self.dim), 0.0).to(device)
            fn = affine_2d if self.dim == 2 else affine_3d
            self.tmp_params = fn(coarse.contiguous().to(device).unsqueeze(0), rois, tuple(self.image_shape), 1, 1,
                                 True, self.SPLINE_ORDER).squeeze(0)
        return self.tmp_params

    def elastic_transform(self, image: torch.Tensor, order=1):
        field = self.dense_field(image.device)
        if order == 0:
            image = image.to(self.img_type)
        fn = apply_offset_2d if self.dim == 2 else apply_offset_3d
        image = fn(image.unsqueeze(0), field.unsqueeze(0), order=order).squeeze(0)
        return image.int() if order == 0 else image

    def apply_to_img(self, result):
        for key in result.get('img_fields', []):
            result[key] = self.elastic_transform(result[key])

    def apply_to_seg(self, result):
        for key in result.get('seg_fields', []):
            result[key] = self.elastic_transform(result[key], order=0)

    def apply_to_det(self, result):
        for _ in result.get('det_fields', []):
            raise NotImplementedError


class CudaCropRandomWithAffine(CudaAugBase):
    """A ``patch_size`` crop at a random position with a random scale / shift / z-rotation, in one
    resample; ``times`` > 1 turns one sample into ``times`` crops (a list of results)."""

    def __init__(self, patch_size, scale, shift, rotate, sampling_ratio=1, order=1, times=1):
        super().__init__()
        self.always = True
        self.dim = len(patch_size)
        self.patch_size = patch_size
        self.scale = scale
        self.shift = shift
        self.rotate = rotate
        self.sampling_ratio = sampling_ratio
        self.order = order
        self.times = times

    def __repr__(self):
        return self.__class__.__name__ + "(patch_size={})".format(self.patch_size)

    @property
    def repeats(self):
        return self.times

    def _forward_params(self, result):
        self._init_params(result)
        start, end = self._forward_crop_params(result)
        scales, shifts, rotate = self._forward_affine_params(result)
        self.params = {"start": start[::-1], "end": end[::-1],  # xyz
                       "_scales": scales, "_shifts": shifts, "_rotate": rotate}
        result[self.key_name] = self.params

    def _check_fit(self):
        assert self.dim == len(self.patch_size)
        assert all(self.image_shape[i] >= self.patch_size[i] for i in range(self.dim)), self.image_shape

    def _forward_crop_params(self, result):
        self._check_fit()
        start = tuple(np.random.randint(0, a - da + 1) for a, da in zip(self.image_shape, self.patch_size))
        return start, tuple(a + b for a, b in zip(start, self.patch_size))

    def _forward_affine_params(self, result):
        scales = [self.get_range(self.scale, 1), ] * self.dim
        shifts = [self.get_range(self.shift, 0) for _ in range(self.dim)]
        rotate = [math.pi * self.get_range(self.rotate, 0) / 180]
        return scales, shifts, rotate

    def _rois(self):
        start = torch.FloatTensor(self.params["start"])
        end = torch.FloatTensor(self.params["end"])
        return _one_roi(self.dim, (start + end) / 2, end - start, torch.FloatTensor(self.params["_shifts"]),
                        torch.FloatTensor(self.params["_scales"]), float(self.params["_rotate"][0]))

    def apply_to_img(self, result):
        _resample_sample(result, self.dim, self._rois(), self.patch_size, self.sampling_ratio, self.order)

    def apply_to_seg(self, result):
        pass  # done together with the images


class CudaCropCenterWithAffine(CudaCropRandomWithAffine):
    def _forward_crop_params(self, result):
        self._check_fit()
        start = tuple(a // 2 - da // 2 for a, da in zip(self.image_shape, self.patch_size))
        return start, tuple(a + b for a, b in zip(start, self.patch_size))


class CudaCropFirstDetWithAffine(CudaCropRandomWithAffine):
    """The crop keeps the first ground-truth box (``result['gt_det'][0]`` = [x1, y1, (z1,) x2, y2, (z2,) ...])
    at least ``border`` voxels inside the patch where the image allows it; random otherwise."""

    def __init__(self, border=12, *args, **kwargs):
        self.border = border
        super().__init__(*args, **kwargs)

    def _forward_crop_params(self, result):
        self._check_fit()
        assert 'gt_det' in result.keys(), "it only used for detection tasks"
        if len(result['gt_det']) == 0:
            return super()._forward_crop_params(result)
        box = result['gt_det'][0].cpu().numpy()
        start = []
        for axis in range(self.dim):  # d, h, w order; the box is xyz
            lo, hi = box[self.dim - axis - 1], box[2 * self.dim - axis - 1]
            room = self.image_shape[axis] - self.patch_size[axis]
            first = min(max(hi + self.border - self.patch_size[axis], 0), room)
            last = min(max(lo - self.border, 0), room)
            start.append(np.random.randint(min(first, last), max(first, last) + 1))
        start = tuple(start)
        return start, tuple(a + b for a, b in zip(start, self.patch_size))
