"""RoIAlignRotated, 2D and 3D, with autograd.

Same public surface as medvision/ops/roi_align_rotated_nd.py: ``RoIAlignRotated2DFunction``,
``RoIAlignRotated3DFunction``, ``roi_align_rotated_2d``, ``roi_align_rotated_3d`` and the
``RoIAlignRotated`` module
(``RoIAlignRotated(output_size, spatial_scale, sampling_ratio=-1, aligned=True)(features, rois, order=1)``).
"""
import torch.nn as nn
from torch.autograd import Function

from .. import _C
from ._common import parse_output_size


def _make_function(ndim):
    fwd = _C.roi_align_rotated_2d_forward if ndim == 2 else _C.roi_align_rotated_3d_forward
    bwd = _C.roi_align_rotated_2d_backward if ndim == 2 else _C.roi_align_rotated_3d_backward

    class _RoIAlignRotatedFunction(Function):
        @staticmethod
        def forward(ctx, features, rois, output_size, spatial_scale, sampling_ratio=0, aligned=True, order=1):
            out = parse_output_size(output_size, ndim)
            ctx.spatial_scale = spatial_scale
            ctx.sampling_ratio = sampling_ratio
            ctx.aligned = aligned
            ctx.order = order
            ctx.save_for_backward(rois)
            ctx.feature_size = features.size()
            assert features.dim() == ndim + 2
            output = features.new_empty((rois.size(0), features.size(1)) + tuple(out))
            fwd(features, rois, output, *out, spatial_scale, sampling_ratio, aligned, order)
            return output

        @staticmethod
        def backward(ctx, grad_output):
            rois = ctx.saved_tensors[0]
            assert ctx.feature_size is not None
            grad_input = None
            if ctx.needs_input_grad[0]:
                grad_input = rois.new_zeros(ctx.feature_size)
                bwd(grad_output.contiguous(), rois, grad_input, *grad_output.shape[2:],
                    ctx.spatial_scale, ctx.sampling_ratio, ctx.aligned, ctx.order)
            return grad_input, None, None, None, None, None, None

    _RoIAlignRotatedFunction.__name__ = f"RoIAlignRotated{ndim}DFunction"
    _RoIAlignRotatedFunction.__qualname__ = _RoIAlignRotatedFunction.__name__
    return _RoIAlignRotatedFunction


RoIAlignRotated2DFunction = _make_function(2)
RoIAlignRotated3DFunction = _make_function(3)
roi_align_rotated_2d = RoIAlignRotated2DFunction.apply
roi_align_rotated_3d = RoIAlignRotated3DFunction.apply


class RoIAlignRotated(nn.Module):
    """RoI align pooling for rotated proposals.

    features: (N, C, H, W) or (N, C, D, H, W); rois: (n, 6) =
    (batch_index, center_x, center_y, w, h, angle) or (n, 10) =
    (batch_index, center_x, center_y, center_z, w, h, d, angle_x, angle_y, angle_z), angles in
    radians, same dtype and device as the features.  In 3D the sample lattice of the roi is
    rotated by Rz(angle_z) * Ry(angle_y) * Rx(angle_x) about the roi centre.

    Args:
        output_size (tuple): (h, w) or (d, h, w); its length selects 2D or 3D
        spatial_scale (float): centre and size are multiplied by this number
        sampling_ratio (int): sub-samples per output bin and axis; <= 0 samples adaptively
        aligned (bool): True shifts the scaled centre by -0.5 so that pixel centres sit at
            half-integer continuous coordinates (the detectron2 convention) and does not clamp
            the roi size; False keeps the legacy convention and forces sizes to >= 1
    """

    def __init__(self, output_size, spatial_scale, sampling_ratio=-1, aligned=True):
        super().__init__()
        assert iter(output_size)
        self.output_size = output_size
        self.spatial_scale = float(spatial_scale)
        self.sampling_ratio = int(sampling_ratio)
        self.aligned = aligned
        self.dim = len(self.output_size)
        if self.dim == 2:
            self.roi_align = roi_align_rotated_2d
        elif self.dim == 3:
            self.roi_align = roi_align_rotated_3d
        else:
            raise Exception("Tried to init RoIAlign module with incorrect output size: {}".format(self.output_size))

    def forward(self, features, rois, order=1):
        assert order in [0, 1], "only support order = 0 (nearest) or 1 (linear)"
        sampling_ratio = 1 if order == 0 else self.sampling_ratio
        return self.roi_align(features, rois, self.output_size, self.spatial_scale, sampling_ratio,
                              self.aligned, order)
