"""RoIAlign (axis-aligned), 2D and 3D, with autograd.

Same public surface as medvision/ops/roi_align_nd.py: ``RoIAlign2DFunction``,
``RoIAlign3DFunction``, ``roi_align_2d``, ``roi_align_3d`` and the ``RoIAlign`` module
(``RoIAlign(output_size, spatial_scale, sampling_ratio=-1)(features, rois, order=1)``).
"""
import torch.nn as nn
from torch.autograd import Function

from .. import _C
from ._common import parse_output_size


def _make_function(ndim):
    fwd = _C.roi_align_2d_forward if ndim == 2 else _C.roi_align_3d_forward
    bwd = _C.roi_align_2d_backward if ndim == 2 else _C.roi_align_3d_backward

    class _RoIAlignFunction(Function):
        @staticmethod
        def forward(ctx, features, rois, output_size, spatial_scale, sampling_ratio=0, order=1):
            out = parse_output_size(output_size, ndim)
            ctx.spatial_scale = spatial_scale
            ctx.sampling_ratio = sampling_ratio
            ctx.order = order
            ctx.save_for_backward(rois)
            ctx.feature_size = features.size()
            assert features.dim() == ndim + 2
            # every element is written by the kernel, so no zero fill is needed
            output = features.new_empty((rois.size(0), features.size(1)) + tuple(out))
            fwd(features, rois, output, *out, spatial_scale, sampling_ratio, order)
            return output

        @staticmethod
        def backward(ctx, grad_output):
            rois = ctx.saved_tensors[0]
            assert ctx.feature_size is not None
            grad_input = None
            if ctx.needs_input_grad[0]:
                # dtype of the rois, as medvision/ops/roi_align_nd.py:62 (rois.new_zeros)
                grad_input = rois.new_zeros(ctx.feature_size)
                bwd(grad_output.contiguous(), rois, grad_input, *grad_output.shape[2:],
                    ctx.spatial_scale, ctx.sampling_ratio, ctx.order)
            return grad_input, None, None, None, None, None

    _RoIAlignFunction.__name__ = f"RoIAlign{ndim}DFunction"
    _RoIAlignFunction.__qualname__ = _RoIAlignFunction.__name__
    return _RoIAlignFunction


RoIAlign2DFunction = _make_function(2)
RoIAlign3DFunction = _make_function(3)
roi_align_2d = RoIAlign2DFunction.apply
roi_align_3d = RoIAlign3DFunction.apply


class RoIAlign(nn.Module):
    """RoI align pooling for axis-aligned proposals.

    features: (N, C, H, W) or (N, C, D, H, W); rois: (n, 5) = (batch_index, x1, y1, x2, y2)
    or (n, 7) = (batch_index, x1, y1, z1, x2, y2, z2), same dtype and device as the features.

    Args:
        output_size (tuple): (h, w) or (d, h, w); its length selects 2D or 3D
        spatial_scale (float): the boxes are multiplied by this number
        sampling_ratio (int): sub-samples per output bin and axis; <= 0 samples adaptively,
            ceil(roi_size / output_size) per axis
    """

    def __init__(self, output_size, spatial_scale, sampling_ratio=-1):
        super().__init__()
        assert iter(output_size)
        self.output_size = output_size
        self.spatial_scale = float(spatial_scale)
        self.sampling_ratio = int(sampling_ratio)
        self.dim = len(self.output_size)
        if self.dim == 2:
            self.roi_align = roi_align_2d
        elif self.dim == 3:
            self.roi_align = roi_align_3d
        else:
            raise Exception("Tried to init RoIAlign module with incorrect output size: {}".format(self.output_size))

    def forward(self, features, rois, order=1):
        assert order in [0, 1], "only support order = 0 (nearest) or 1 (linear)"
        # nearest neighbour takes one sample per bin: averaging samples would blend labels
        sampling_ratio = 1 if order == 0 else self.sampling_ratio
        return self.roi_align(features, rois, self.output_size, self.spatial_scale, sampling_ratio, order)
