"""Sliding-window patch extraction for inference: many rois on one image.

``CudaPatches`` of medvision/aug_cuda/aug_testtime.py:10-150 (anchor grid :44-67, roi
construction and the ``affine_*`` call :77-150) on a single (C, [D,] H, W) CUDA sample.  As in the
reference, the backward pass only takes the anchor list back out of ``result``
(aug_testtime.py:69-73): the reference's stitching of image / label patches is commented out
(:152 onwards) and only its detection boxes are mapped back.  That detection-box bookkeeping
(cropBBoxes / padBBoxes / NMS) is not part of the resampling path and is not provided.
"""
import numpy as np
import torch

from .base import CudaAugBase
from ..ops.cuda_fun_tools import affine_2d, affine_3d


class CudaPatches(CudaAugBase):
    """ONLY FOR INFERENCE OR EVALUATION: cuts the image into overlapping patches.

    result['img'] is (C, [D,] H, W); the patches of field ``key`` are stored under
    ``'patches_' + key`` with shape (n_patches, C, *patch_size) (the sample is passed as a batch of
    one; a single patch loses its leading axis, as ``.squeeze(0)`` does in the reference)."""

    def __init__(self, patch_size=(128, 128), overlap=0.5, fusion_mode='max'):
        super().__init__()
        assert fusion_mode in ('max', 'mean', 'src')
        self.always = True
        self.patch_size = tuple(patch_size)
        self.overlap = overlap
        self.fusion_mode = fusion_mode
        self._stride = [p - int(p * overlap) for p in patch_size]
        self._base_anchor = [0] * len(patch_size) + list(patch_size)  # zyx

    def __repr__(self):
        return self.__class__.__name__ + '(patch_size={}, overlap={}, fusion_mode={})'.format(
            self.patch_size, self.overlap, self.fusion_mode)

    @property
    def canBackward(self):
        return True

    def _forward_params(self, result):
        self._init_params(result)
        assert len(self.patch_size) == self.dim
        grid = [np.arange(max((s - 1) // self._stride[i], 1)) * self._stride[i]
                for i, s in enumerate(self.image_shape)]  # zyx
        ctr = np.meshgrid(*grid, indexing='ij')
        ctr = np.stack([*ctr] * 2, axis=0)
        axes = list(range(1, self.dim + 1))
        anchors = ctr + np.expand_dims(self._base_anchor, axis=axes)  # [z,y,x,z,y,x] per grid point
        anchors = np.transpose(anchors, tuple(axes + [0])).reshape([-1, 2 * self.dim])
        anchors = anchors[:, [2, 1, 0, 5, 4, 3]] if self.dim == 3 else anchors[:, [1, 0, 3, 2]]  # -> xyz
        self.params = anchors
        result[self.key_name] = self.params

    def _backward_params(self, result):
        self._init_params(result)
        params = result.pop(self.key_name, None)
        if params is not None:
            self.params = np.array(params)

    def _rois(self):
        n = len(self.params)
        index = torch.zeros(n, 1)
        boxes = torch.FloatTensor(self.params)  # xyz start, xyz end
        center = boxes[:, :self.dim] / 2 + boxes[:, self.dim:] / 2
        shape = boxes[:, self.dim:] - boxes[:, :self.dim]
        angles = torch.zeros(n, 1 if self.dim == 2 else 3)
        return torch.cat([index, center, shape, angles], dim=1)

    def apply_to_img(self, result):
        if not self.isForwarding:
            return  # nothing is stitched back, as in the reference
        fn = affine_2d if self.dim == 2 else affine_3d
        rois = self._rois()
        for key in result.get('img_fields', []):
            image = result[key]
            patches = fn(image.unsqueeze(0), rois.to(image.device), self.patch_size, 1, 1, True, 1)
            result[f'patches_{key}'] = patches.squeeze(0)
        for key in result.get('seg_fields', []):
            image = result[key]
            src = image if image.is_floating_point() and image.dtype != torch.float64 else image.float()
            patches = fn(src.unsqueeze(0), rois.to(image.device), self.patch_size, 1, 1, True, 0)
            result[f'patches_{key}'] = patches.squeeze(0).to(image.dtype)
