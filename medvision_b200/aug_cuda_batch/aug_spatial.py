"""Batched geometric augmentations built on the resampling op.

Same classes, constructor arguments, parameter draws and roi formulas as the resampling
transforms of medvision/aug_cuda_batch/aug_spatial.py (Resize :69-194, RandomAffine / Scale /
Shift / Rotate :355-597, Crop*WithAffine :600-957).  What differs:
  * the rois of a call are built once (float32 on the host, in the reference's operation order,
    so the values are the same) and shared by the image and the label fields;
  * ``times`` crops per image address the SAME image through the roi's batch index instead of
    concatenating ``times`` copies of the batch;
  * label fields go through the nearest-neighbour path of the same kernel.
"""
import math
import random
from typing import Union

import numpy as np
import torch

from .base import BatchCudaAugBase
from ..ops.cuda_fun_tools import (affine_2d, affine_3d, affine_fields_3d, affine_label_2d, affine_label_3d,
                                  apply_offset_2d, apply_offset_3d)
from ..ops.roi_stage import stage_rois


def _resample_fields(result, dim, rois, out_size, sampling_ratio, order):
    """All image and label fields of ``result`` through the rois of this call (CPU float32).  The rois go to the
    device once (one asynchronous copy, float32 and float16 at once); in 3D an image field and a label field are
    resampled by one fused call whose label work rides along with the image's launches."""
    out_size = tuple(int(v) for v in out_size)
    assert not result.get('det_fields'), 'detection boxes are not handled by the resampling transforms'
    img_keys, seg_keys = list(result.get('img_fields', [])), list(result.get('seg_fields', []))
    fields = [result[k] for k in img_keys + seg_keys]
    if not fields:
        return
    for image in fields:
        assert image.is_cuda, 'image should be cuda'
        assert image.ndim == dim + 2, 'image should be batch, channel, **dim'
    device = fields[0].device
    rois_f32, rois_f16, release = stage_rois(rois, device)

    def rois_for(t):
        r = rois_f16 if t.dtype == torch.float16 else rois_f32
        return r if t.device == device else r.to(t.device, non_blocking=True)

    fn = affine_2d if dim == 2 else affine_3d
    label_fn = affine_label_2d if dim == 2 else affine_label_3d
    fused = 0
    if dim == 3 and sampling_ratio == 1 and order in (0, 1):  # pairs of (image field, label field): one call each
        for ik, sk in zip(img_keys, seg_keys):
            image, seg = result[ik], result[sk]
            if image.device != device or seg.device != device or image.shape[0] != seg.shape[0] \
                    or image.shape[2:] != seg.shape[2:] or image.dtype not in (torch.float16, torch.float32):
                break
            result[ik], result[sk] = affine_fields_3d(image, seg, rois_f32, out_size, 1.0, True, order,
                                                      rois_image=rois_for(image))
            fused += 1
    for key in img_keys[fused:]:
        image = result[key]
        result[key] = fn(image, rois_for(image), out_size, 1.0, sampling_ratio, True, order)
    for key in seg_keys[fused:]:
        image = result[key]
        # = fn(image.float(), rois, out_size, 1.0, 1, True, 0).int() of the reference, on the integers themselves
        r = rois_f32 if image.device == device else rois_f32.to(image.device, non_blocking=True)
        result[key] = label_fn(image, r, out_size, 1.0, True)
    release()


def _affine_rois(index, center, shape, shifts, scales, rotate, dim):
    """[index, center - shape * shifts / scales, shape / scales, angles]; rotation about z in 3D."""
    if dim == 2:
        angles = rotate
    else:
        angles = torch.cat([torch.zeros_like(rotate), torch.zeros_like(rotate), rotate], dim=1)
    return torch.cat([index, center - shape * shifts / scales, shape / scales, angles], dim=-1)


class BatchCudaResize(BatchCudaAugBase):
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
        index = torch.arange(self.batch, dtype=torch.float32).unsqueeze(-1)
        center = torch.tensor([i / 2 for i in self.image_shape[::-1]], dtype=torch.float32)  # dhw => xyz
        shape = torch.tensor(list(self.image_shape[::-1]), dtype=torch.float32)
        angles = torch.zeros(1 if self.dim == 2 else 3)
        boxes = torch.cat([center, shape, angles]).unsqueeze(0).repeat(self.batch, 1)
        return torch.cat([index, boxes], dim=-1)

    def apply_to_img(self, result):
        # the whole image is one roi; image and label fields share it
        if all(i == 1.0 for i in self.params):
            return
        out_size = tuple(int(i * p) for i, p in zip(self.image_shape, self.params))
        _resample_fields(result, self.dim, self._rois(), out_size, 1, self.order)

    def apply_to_seg(self, result):
        pass  # done together with the images


class BatchCudaRandomAffine(BatchCudaAugBase):
    def __init__(self, p, scale: Union[float, list, tuple], shift: Union[float, list, tuple],
                 rotate: Union[float, list, tuple], sampling_ratio=1, order=1):
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

    def _forward_params(self, result):
        self._init_params(result)
        scales, shifts, rotate = [], [], []
        for _ in range(self.batch):
            scales.append([self.get_range(self.scale, 1), ] * self.dim)
            shifts.append([self.get_range(self.shift, 0) for _ in range(self.dim)])
            rotate.append([math.pi * self.get_range(self.rotate, 0) / 180])
        self.params = {"scales": np.array(scales), "shifts": np.array(shifts), "rotate": np.array(rotate)}
        result[self.key_name] = self.params

    def _backward_params(self, result: dict):
        self._init_params(result)
        params = result.get(self.key_name, None)
        if params:
            self.params = {"scales": 1 / params["scales"], "shifts": -params["shifts"], "rotate": -params["rotate"]}

    def _rois(self):
        scales = torch.FloatTensor(self.params["scales"])
        shifts = torch.FloatTensor(self.params["shifts"])
        rotate = torch.FloatTensor(self.params["rotate"])
        index = torch.arange(self.batch, dtype=torch.float32).unsqueeze(-1)
        center = torch.tensor([i / 2 for i in self.image_shape[::-1]], dtype=torch.float32)
        shape = torch.tensor(list(self.image_shape[::-1]), dtype=torch.float32)
        return _affine_rois(index, center, shape, shifts, scales, rotate, self.dim)

    def apply_to_img(self, result: dict):
        _resample_fields(result, self.dim, self._rois(), self.image_shape, self.sampling_ratio, self.order)

    def apply_to_seg(self, result: dict):
        pass  # done together with the images


class BatchCudaRandomScale(BatchCudaRandomAffine):
    def __init__(self, p, scale: Union[float, list, tuple], sampling_ratio=1):
        super().__init__(p, scale=scale, shift=0, rotate=0, sampling_ratio=sampling_ratio)


class BatchCudaRandomShift(BatchCudaRandomAffine):
    def __init__(self, p, shift: Union[float, list, tuple], sampling_ratio=1):
        super().__init__(p, scale=0, shift=shift, rotate=0, sampling_ratio=sampling_ratio)


class BatchCudaRandomRotate(BatchCudaRandomAffine):
    def __init__(self, p, rotate: Union[float, list, tuple], sampling_ratio=1):
        super().__init__(p, scale=0, shift=0, rotate=rotate, sampling_ratio=sampling_ratio)


class BatchCudaRandomElasticDeformation(BatchCudaAugBase):
    """Random smooth warp, as medvision/aug_cuda_batch/aug_spatial.py:204-313: a coarse grid of
    ``num_control_points`` random displacements per sample (at most ``max_displacement`` half grid
    cells, the two outermost control points of every axis locked to zero) is blown up to a dense
    (B, dim, *image_shape) field by one ``affine_*`` resample (order ``order``, Catmull-Rom by
    default) and applied with ``apply_offset_*``: linear for images, nearest for labels.  The dense
    field is built once per call and shared by all fields; ``backward`` negates the coarse field."""

    def __init__(self, p, num_control_points=8, max_displacement: float = 0.8, order=3):
        super().__init__()
        self.p = p
        self.num_control_points = num_control_points  # d, h, w order
        self.max_displacement = max_displacement
        self.INTER_ORDER = order
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
        fields = []
        for _ in range(self.batch):
            coarse = 2 * np.random.rand(*grid_shape, self.dim).astype(np.float32) - 1  # [-1, 1)
            coarse *= reach.astype(np.float32)
            for axis in range(self.dim):
                locked = [slice(None)] * self.dim
                for i in range(self.num_locked_borders):
                    for pos in (i, -1 - i):
                        locked[axis] = pos
                        coarse[tuple(locked)] = 0
            fields.append(coarse)
        self.params = np.array(fields)
        result[self.key_name] = self.params

    def _backward_params(self, result):
        self.tmp_params = None
        self._init_params(result)
        params = result.pop(self.key_name, None)
        if params is not None:
            self.params = -params

    def dense_field(self, device):
        """(B, dim, *image_shape) float32 displacement field on ``device``."""
        if self.tmp_params is None:
            # channels first; halved to smooth
            coarse = torch.from_numpy(self.params).permute(0, self.dim + 1, *range(1, self.dim + 1)) / 2
            grid = coarse.shape[2:]
            index = torch.arange(self.batch, dtype=torch.float32).unsqueeze(-1)
            center = torch.tensor([i / 2 for i in grid[::-1]], dtype=torch.float32)
            shape = torch.tensor(list(grid[::-1]), dtype=torch.float32) - (2 * self.num_locked_borders - 1)
            angles = torch.zeros(1 if self.dim == 2 else 3)
            boxes = torch.cat([center, shape, angles]).unsqueeze(0).repeat(self.batch, 1)
            rois = torch.cat([index, boxes], dim=-1).to(device)
            fn = affine_2d if self.dim == 2 else affine_3d
            self.tmp_params = fn(coarse.contiguous().to(device), rois, tuple(self.image_shape), 1, 1, True,
                                 self.INTER_ORDER)
        return self.tmp_params

    def elastic_transform(self, image: torch.Tensor, order=1):
        field = self.dense_field(image.device)
        if order == 0:
            image = image.to(self.img_type)
        image = (apply_offset_2d if self.dim == 2 else apply_offset_3d)(image, field, order=order)
        if order == 0:
            image = image.int()
        return image

    def apply_to_img(self, result):
        for key in result.get('img_fields', []):
            result[key] = self.elastic_transform(result[key])

    def apply_to_seg(self, result):
        for key in result.get('seg_fields', []):
            result[key] = self.elastic_transform(result[key], order=0).int()

    def apply_to_det(self, result):
        for key in result.get('det_fields', []):
            raise NotImplementedError


class BatchCudaCropRandomWithAffine(BatchCudaAugBase):
    def __init__(self, patch_size, scale: Union[float, list, tuple], shift: Union[float, list, tuple],
                 rotate: Union[float, list, tuple], sampling_ratio=1, order=1, times=1):
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

    def _init_params(self, result):
        super()._init_params(result)
        self.n_images = self.batch
        self.batch = self.n_images * self.times  # one parameter set per produced patch

    def _forward_params(self, result):
        self._init_params(result)
        assert self.dim == len(self.patch_size)
        assert all(self.image_shape[i] >= self.patch_size[i] for i in range(self.dim)), self.image_shape
        batch_start, batch_end = self._forward_crop_params(result)
        batch_scales, batch_shifts, batch_rotate = self._forward_affine_params(result)
        self.params = {"start": batch_start, "end": batch_end,  # xyz
                       "scales": batch_scales, "shifts": batch_shifts, "rotate": batch_rotate}
        result[self.key_name] = self.params

    def _forward_affine_params(self, result: dict):
        scales, shifts, rotate = [], [], []
        for _ in range(self.batch):
            scales.append([self.get_range(self.scale, 1), ] * self.dim)
            shifts.append([self.get_range(self.shift, 0) for _ in range(self.dim)])
            rotate.append([math.pi * self.get_range(self.rotate, 0) / 180])
        return np.array(scales), np.array(shifts), np.array(rotate)

    def _random_start(self):
        return tuple(map(lambda a, da: np.random.randint(0, a - da + 1), self.image_shape, self.patch_size))

    def _start_near(self, obj):
        """a patch start such that the patch covers the object ``obj`` (slices, dhw) with a border"""
        lo = tuple(min(max(obj[d].stop + self.border - self.patch_size[d], 0), self.image_shape[d] - self.patch_size[d])
                   for d in range(len(obj)))
        hi = tuple(min(max(obj[d].start - self.border, 0), self.image_shape[d] - self.patch_size[d])
                   for d in range(len(obj)))
        return tuple(map(lambda a, da: np.random.randint(min(a, da), max(a, da) + 1), lo, hi))

    def _collect(self, starts):
        batch_start = [s[::-1] for s in starts]
        batch_end = [tuple(a + b for a, b in zip(s, self.patch_size))[::-1] for s in starts]
        return np.array(batch_start), np.array(batch_end)

    def _forward_crop_params(self, result: dict):
        return self._collect([self._random_start() for _ in range(self.batch)])

    def _rois(self):
        start = torch.FloatTensor(self.params["start"])
        end = torch.FloatTensor(self.params["end"])
        scales = torch.FloatTensor(self.params["scales"])
        shifts = torch.FloatTensor(self.params["shifts"])
        rotate = torch.FloatTensor(self.params["rotate"])
        # patch r*B + b is cut from image b
        index = (torch.arange(self.batch) % self.n_images).float().unsqueeze(-1)
        return _affine_rois(index, (start + end) / 2, end - start, shifts, scales, rotate, self.dim)

    def apply_to_img(self, result: dict):
        _resample_fields(result, self.dim, self._rois(), self.patch_size, self.sampling_ratio, self.order)

    def apply_to_seg(self, result: dict):
        pass  # done together with the images


class BatchCudaCropCenterWithAffine(BatchCudaCropRandomWithAffine):
    def _forward_crop_params(self, result: dict):
        start = tuple(map(lambda a, da: a // 2 - da // 2, self.image_shape, self.patch_size))
        return self._collect([start for _ in range(self.batch)])


class BatchCudaCropForegroundWithAffine(BatchCudaCropRandomWithAffine):
    def __init__(self, border=12, **kwargs):
        super().__init__(**kwargs)
        self.border = border

    def _forward_crop_params(self, result: dict):
        import scipy.ndimage as ndi
        assert 'gt_seg' in result.keys() or 'pseudo_mask' in result.keys()
        mask = result['gt_seg'] if 'gt_seg' in result.keys() else result['pseudo_mask']
        starts = []
        for i in range(self.batch):
            foreground = mask[i % self.n_images, 0]
            if torch.is_tensor(foreground):
                foreground = foreground.cpu().numpy()
            objs = ndi.find_objects(ndi.label(foreground)[0])
            starts.append(self._start_near(random.choice(objs)) if len(objs) else self._random_start())
        return self._collect(starts)


class BatchCudaCropDetWithAffine(BatchCudaCropRandomWithAffine):
    """patches around the ground-truth boxes, one box after the other over the repeats"""

    def __init__(self, border=12, **kwargs):
        super().__init__(**kwargs)
        self.border = border
        self.current_repeat_idx = 0

    def _box(self, result, k):
        obj = result['gt_det'][k]
        return [slice(int(obj[self.dim - i - 1]), int(obj[2 * self.dim - i - 1])) for i in range(self.dim)]

    def _forward_crop_params(self, result: dict):
        assert 'gt_det' in result.keys(), "it only used for detection tasks"
        starts = []
        for _ in range(self.batch):
            k = min(self.current_repeat_idx % self.repeats, len(result['gt_det']) - 1)
            self.current_repeat_idx += 1
            starts.append(self._start_near(self._box(result, k)))
        return self._collect(starts)


class BatchCudaCropFirstDetWithAffine(BatchCudaCropDetWithAffine):
    def _forward_crop_params(self, result: dict):
        assert 'gt_det' in result.keys(), "it only used for detection tasks"
        return self._collect([self._start_near(self._box(result, 0)) for _ in range(self.batch)])
