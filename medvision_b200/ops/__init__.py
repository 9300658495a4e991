from .roi_align_nd import RoIAlign
from .roi_align_rotated_nd import RoIAlignRotated
from .cuda_fun_tools import (affine_2d, affine_3d, affine_fields_3d, affine_label_2d, affine_label_3d,
                             apply_offset_2d, apply_offset_3d)
from .host_pipeline import affine_from_host

__all__ = ['RoIAlign', 'RoIAlignRotated', 'affine_2d', 'affine_3d', 'affine_from_host', 'apply_offset_2d', 'apply_offset_3d', 'affine_label_2d',
           'affine_label_3d', 'affine_fields_3d']
