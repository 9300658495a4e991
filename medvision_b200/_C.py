"""The ten resampling functions of the reference's compiled extension, on torch tensors.

Same names, argument order and error behaviour as ``medvision._C``
(medvision/csrc/vision.cpp:34-48,74-75 and the dispatch headers medvision/csrc/roi_align_*.h,
affine_*.h): every function returns ``None`` and writes into a caller-allocated tensor;
a non-CUDA input raises ``RuntimeError("... is not implemented on CPU")``; a wrong roi width
raises ``RuntimeError("wrong roi size! size_rois should be K")``.

Differences from the reference, all deliberate: the launch goes to torch's CURRENT stream of
the input's device under a device guard (the reference launches on the legacy default stream of
whatever device is current); flat offsets are 64-bit; an empty roi list is a no-op (the reference
fails with a zero-block launch); a roi whose batch index lies outside the batch yields zeros and
sets a status bit (see :func:`last_status`) instead of reading out of bounds.
"""
import torch

from . import _lib

_DTYPES = {torch.float32: _lib.MVR_F32, torch.float16: _lib.MVR_F16, torch.float64: _lib.MVR_F64}
_status_words = {}


def _status_ptr(device):
    w = _status_words.get(device.index)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device.index] = w
    return w.data_ptr()


def last_status(device=None, clear=True):
    """Status bits OR-ed by the kernels launched on ``device`` so far (synchronises)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _status_words.get(device.index if device.index is not None else torch.cuda.current_device())
    if w is None:
        return 0
    v = int(w.item())
    if clear:
        w.zero_()
    return v


def _dtype_code(t, what):
    code = _DTYPES.get(t.dtype)
    if code is None:
        # AT_DISPATCH_FLOATING_TYPES_AND_HALF message of the reference's launchers
        raise RuntimeError(f'"{what}" not implemented for \'{str(t.dtype).replace("torch.", "")}\'')
    return code


def _check(op, data, rois, other, size_rois):
    if not data.is_cuda:
        raise RuntimeError(f"{op} is not implemented on CPU")
    if rois.dim() != 2 or rois.size(1) != size_rois:
        raise RuntimeError(f"wrong roi size! size_rois should be {size_rois}")
    if not (rois.is_cuda and other.is_cuda) or rois.device != data.device or other.device != data.device:
        raise RuntimeError("expected all tensors to be on the same CUDA device")
    if rois.dtype != data.dtype or other.dtype != data.dtype:
        # the reference reinterprets with tensor.data<scalar_t>(), which throws on a mismatch
        raise RuntimeError(f"expected scalar type {data.dtype} but found {rois.dtype if rois.dtype != data.dtype else other.dtype}")


def _call(fn, *args):
    rc = fn(*args)
    if rc != 0:
        raise RuntimeError(_lib.strerror(rc))


def _run(name, op, ndim, kind_width, a, rois, b, out_sizes, spatial_scale, sampling_ratio, aligned, order, forward):
    """a: features (fwd) or top_grad (bwd); b: output (fwd) or bottom_grad (bwd)."""
    feat = a if forward else b
    _check(op, a, rois, b, kind_width)
    code = _dtype_code(a, name)
    if feat.dim() != ndim + 2:
        raise RuntimeError(f"{name}: expected a {ndim + 2}-D feature tensor")
    a_c = a.contiguous()
    rois_c = rois.contiguous()
    if not b.is_contiguous():
        raise RuntimeError(f"{name}: the result tensor must be contiguous")
    N, C = feat.size(0), feat.size(1)
    spatial = list(feat.shape[2:])
    R = rois.size(0)
    expect = (R, C) + tuple(out_sizes)
    other = b if forward else a
    if tuple(other.shape) != expect:
        raise RuntimeError(f"{name}: expected a tensor of shape {expect}, got {tuple(other.shape)}")
    fn = getattr(_lib.lib, "mvr_" + name)
    with torch.cuda.device(a.device):
        stream = torch.cuda.current_stream(a.device).cuda_stream
        args = [a_c.data_ptr(), rois_c.data_ptr(), b.data_ptr(), code, N, C] + spatial + [R, rois.size(1)] + \
               list(out_sizes) + [float(spatial_scale), int(sampling_ratio)]
        if aligned is not None:
            args.append(int(bool(aligned)))
        args += [int(order), _status_ptr(a.device), stream]
        _call(fn, *args)


def roi_align_2d_forward(input, rois, output, aligned_height, aligned_width, spatial_scale, sampling_ratio, order):
    _run("roi_align_2d_forward", "RoIAlign", 2, 5, input, rois, output, (aligned_height, aligned_width),
         spatial_scale, sampling_ratio, None, order, True)


def roi_align_2d_backward(top_grad, rois, bottom_grad, aligned_height, aligned_width, spatial_scale, sampling_ratio,
                          order):
    _run("roi_align_2d_backward", "RoIAlign", 2, 5, top_grad, rois, bottom_grad, (aligned_height, aligned_width),
         spatial_scale, sampling_ratio, None, order, False)


def roi_align_3d_forward(input, rois, output, aligned_depth, aligned_height, aligned_width, spatial_scale,
                         sampling_ratio, order):
    _run("roi_align_3d_forward", "RoIAlign", 3, 7, input, rois, output,
         (aligned_depth, aligned_height, aligned_width), spatial_scale, sampling_ratio, None, order, True)


def roi_align_3d_backward(top_grad, rois, bottom_grad, aligned_depth, aligned_height, aligned_width, spatial_scale,
                          sampling_ratio, order):
    _run("roi_align_3d_backward", "RoIAlign", 3, 7, top_grad, rois, bottom_grad,
         (aligned_depth, aligned_height, aligned_width), spatial_scale, sampling_ratio, None, order, False)


def roi_align_rotated_2d_forward(input, rois, output, aligned_height, aligned_width, spatial_scale, sampling_ratio,
                                 aligned, order):
    _run("roi_align_rotated_2d_forward", "RoIAlignRotated", 2, 6, input, rois, output,
         (aligned_height, aligned_width), spatial_scale, sampling_ratio, aligned, order, True)


def roi_align_rotated_2d_backward(top_grad, rois, bottom_grad, aligned_height, aligned_width, spatial_scale,
                                  sampling_ratio, aligned, order):
    _run("roi_align_rotated_2d_backward", "RoIAlignRotated", 2, 6, top_grad, rois, bottom_grad,
         (aligned_height, aligned_width), spatial_scale, sampling_ratio, aligned, order, False)


def roi_align_rotated_3d_forward(input, rois, output, aligned_depth, aligned_height, aligned_width, spatial_scale,
                                 sampling_ratio, aligned, order):
    _run("roi_align_rotated_3d_forward", "RoIAlignRotated", 3, 10, input, rois, output,
         (aligned_depth, aligned_height, aligned_width), spatial_scale, sampling_ratio, aligned, order, True)


def roi_align_rotated_3d_backward(top_grad, rois, bottom_grad, aligned_depth, aligned_height, aligned_width,
                                  spatial_scale, sampling_ratio, aligned, order):
    _run("roi_align_rotated_3d_backward", "RoIAlignRotated", 3, 10, top_grad, rois, bottom_grad,
         (aligned_depth, aligned_height, aligned_width), spatial_scale, sampling_ratio, aligned, order, False)


def affine_2d(input, rois, output, aligned_height, aligned_width, spatial_scale, sampling_ratio, aligned, order):
    _run("affine_2d", "RoIAlignRotated", 2, 6, input, rois, output, (aligned_height, aligned_width),
         spatial_scale, sampling_ratio, aligned, order, True)


def affine_3d(input, rois, output, aligned_depth, aligned_height, aligned_width, spatial_scale, sampling_ratio,
              aligned, order):
    _run("affine_3d", "RoIAlignRotated", 3, 10, input, rois, output,
         (aligned_depth, aligned_height, aligned_width), spatial_scale, sampling_ratio, aligned, order, True)
