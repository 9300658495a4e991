"""The resampling functions of the reference's compiled extension, on torch tensors: the ten
roi / affine functions and ``deform_2d`` / ``deform_3d`` in the configuration ``apply_offset_*`` uses.

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


def cached_memory_bytes(device=None):
    """Bytes held by the library's memory pool on ``device`` (the float accumulator volumes of the dense 3D half
    backward come from it; it keeps up to 1 GiB between calls)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    with torch.cuda.device(index):
        return int(_lib.lib.mvr_cached_memory_bytes())


def release_cached_memory(device=None):
    """Give the unused part of that pool back to the driver."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    with torch.cuda.device(index):
        rc = _lib.lib.mvr_release_cached_memory()
    if rc != 0:
        raise RuntimeError(_lib.strerror(rc))


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
    dev = data.device
    if rois.device != dev or other.device != dev:
        raise RuntimeError("expected all tensors to be on the same CUDA device")
    if rois.dtype != data.dtype or other.dtype != data.dtype:
        # the reference reinterprets with tensor.data<scalar_t>(), which throws on a mismatch
        raise RuntimeError(f"expected scalar type {data.dtype} but found {rois.dtype if rois.dtype != data.dtype else other.dtype}")


def _call(fn, *args):
    rc = fn(*args)
    if rc != 0:
        raise RuntimeError(_lib.strerror(rc))


_FN = {name: getattr(_lib.lib, name) for name in _lib.PROTOTYPES}
_raw_stream = torch._C._cuda_getCurrentRawStream  # (device index) -> cudaStream_t of torch's current stream
_current_device = torch._C._cuda_getDevice


def _launch(fn, device, args):
    """Call ``fn(*args, stream)`` with ``device`` current and torch's current stream of that device."""
    index = device.index
    if _current_device() == index:
        rc = fn(*args, _raw_stream(index))
    else:
        with torch.cuda.device(index):
            rc = fn(*args, _raw_stream(index))
    if rc != 0:
        raise RuntimeError(_lib.strerror(rc))


def _run(name, op, ndim, kind_width, a, rois, b, out_sizes, spatial_scale, sampling_ratio, aligned, order, forward):
    """a: features (fwd) or top_grad (bwd); b: output (fwd) or bottom_grad (bwd)."""
    feat = a if forward else b
    _check(op, a, rois, b, kind_width)
    code = _DTYPES.get(a.dtype)
    if code is None:
        _dtype_code(a, name)
    if feat.dim() != ndim + 2:
        raise RuntimeError(f"{name}: expected a {ndim + 2}-D feature tensor")
    if not a.is_contiguous():
        a = a.contiguous()
    if not rois.is_contiguous():
        rois = rois.contiguous()
    if not b.is_contiguous():
        raise RuntimeError(f"{name}: the result tensor must be contiguous")
    fshape = feat.shape
    R = rois.shape[0]
    other = b if forward else a
    if other.shape != (R, fshape[1], *out_sizes):
        raise RuntimeError(f"{name}: expected a tensor of shape {(R, fshape[1], *out_sizes)}, got {tuple(other.shape)}")
    device = a.device
    if aligned is None:
        args = (a.data_ptr(), rois.data_ptr(), b.data_ptr(), code, *fshape, R, kind_width, *out_sizes,
                float(spatial_scale), int(sampling_ratio), int(order), _status_ptr(device))
    else:
        args = (a.data_ptr(), rois.data_ptr(), b.data_ptr(), code, *fshape, R, kind_width, *out_sizes,
                float(spatial_scale), int(sampling_ratio), 1 if aligned else 0, int(order), _status_ptr(device))
    _launch(_FN["mvr_" + name], device, args)


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


_LABEL_DTYPES = {torch.uint8: 0, torch.int16: 1, torch.int32: 2, torch.int64: 3}


def affine_label(input, rois, output, out_sizes, spatial_scale, aligned):
    """Nearest resampling of an integer label tensor into an int32 ``output``: the result of the
    reference's ``affine_*(input.float(), rois, ..., order=0).int()`` without the float copies.
    ``rois`` is float32.  Not a function of the reference's extension.  Returns False when the
    library has no label kernel for the shape (the caller then takes the cast path)."""
    ndim = input.dim() - 2
    if not input.is_cuda:
        raise RuntimeError("RoIAlignRotated is not implemented on CPU")
    code = _LABEL_DTYPES.get(input.dtype)
    if code is None:
        raise RuntimeError(f'"affine_label" not implemented for \'{str(input.dtype).replace("torch.", "")}\'')
    width = 6 if ndim == 2 else 10
    if rois.dim() != 2 or rois.size(1) != width:
        raise RuntimeError(f"wrong roi size! size_rois should be {width}")
    if rois.dtype != torch.float32 or output.dtype != torch.int32:
        raise RuntimeError("affine_label: rois must be float32 and the output int32")
    if rois.device != input.device or output.device != input.device:
        raise RuntimeError("expected all tensors to be on the same CUDA device")
    if not input.is_contiguous():
        input = input.contiguous()
    if not rois.is_contiguous():
        rois = rois.contiguous()
    R = rois.shape[0]
    if not output.is_contiguous() or output.shape != (R, input.shape[1], *out_sizes):
        raise RuntimeError("affine_label: the output must be a contiguous (R, C, *out_size) tensor")
    device = input.device
    index = device.index
    args = (input.data_ptr(), code, rois.data_ptr(), output.data_ptr(), *input.shape, R, width, *out_sizes,
            float(spatial_scale), 1 if aligned else 0, _status_ptr(device))
    fn = _FN["mvr_affine_label_%dd" % ndim]
    with torch.cuda.device(index):
        rc = fn(*args, _raw_stream(index))
    if rc == _lib.MVR_ERR_UNSUPPORTED:
        return False
    if rc != 0:
        raise RuntimeError(_lib.strerror(rc))
    return True


def affine_fields_3d(image, image_rois, image_out, labels, label_rois, label_out, out_sizes, spatial_scale, aligned,
                     order):
    """An image field and its label field of one augmentation call: ``affine_3d(image, image_rois, ...,
    sampling_ratio 1)`` into ``image_out`` and :func:`affine_label` of ``labels`` (float32 ``label_rois``, the same
    rois) into the int32 ``label_out``, with the label's work riding along with the image's launches where the
    shapes allow.  Not a function of the reference's extension."""
    if not (image.is_cuda and labels.is_cuda):
        raise RuntimeError("RoIAlignRotated is not implemented on CPU")
    if image.dim() != 5 or labels.dim() != 5 or image.shape[0] != labels.shape[0] or image.shape[2:] != labels.shape[2:]:
        raise RuntimeError("affine_fields_3d: image and labels must be (N, C, D, H, W) over the same volumes")
    code = _dtype_code(image, "affine_3d")
    lcode = _LABEL_DTYPES.get(labels.dtype)
    if lcode is None or code == _lib.MVR_F64:
        raise RuntimeError("affine_fields_3d: float16 / float32 image and uint8 / int16 / int32 / int64 labels")
    for r in (image_rois, label_rois):
        if r.dim() != 2 or r.size(1) != 10:
            raise RuntimeError("wrong roi size! size_rois should be 10")
    R = image_rois.shape[0]
    if label_rois.shape[0] != R or image_rois.dtype != image.dtype or label_rois.dtype != torch.float32:
        raise RuntimeError("affine_fields_3d: rois in the image's dtype for the image and in float32 for the labels")
    dev = image.device
    for t in (image_rois, image_out, labels, label_rois, label_out):
        if t.device != dev:
            raise RuntimeError("expected all tensors to be on the same CUDA device")
    if image_out.dtype != image.dtype or label_out.dtype != torch.int32:
        raise RuntimeError("affine_fields_3d: image_out in the image's dtype, label_out int32")
    if image_out.shape != (R, image.shape[1], *out_sizes) or label_out.shape != (R, labels.shape[1], *out_sizes) \
            or not image_out.is_contiguous() or not label_out.is_contiguous():
        raise RuntimeError("affine_fields_3d: the results must be contiguous (R, C, *out_size) tensors")
    image, labels = image.contiguous(), labels.contiguous()
    image_rois, label_rois = image_rois.contiguous(), label_rois.contiguous()
    N, _, D, H, W = image.shape
    _launch(_FN["mvr_affine_fields_3d"], dev,
            (image.data_ptr(), code, image_rois.data_ptr(), image_out.data_ptr(), image.shape[1],
             labels.data_ptr(), lcode, label_rois.data_ptr(), label_out.data_ptr(), labels.shape[1],
             N, D, H, W, R, 10, *out_sizes, float(spatial_scale), 1 if aligned else 0, int(order), _status_ptr(dev)))


def apply_offset(input, offset, order):
    """Displacement-field warp: ``out[b, c, p] = interp(input[b, c], p + offset[b, :, p])``.  Not a
    function of the reference's extension: it is what ``deform_2d`` / ``deform_3d`` compute in the
    configuration ``apply_offset_2d/3d`` call them with.  A float32 field with a half image is
    rounded to half as it is read (the reference casts it in a pass of its own)."""
    ndim = input.dim() - 2
    name = "deform_%dd" % ndim
    if not input.is_cuda:
        raise RuntimeError("Not implemented on the CPU")
    if ndim not in (2, 3) or offset.dim() != ndim + 2 or offset.size(1) != ndim or \
            offset.shape[2:] != input.shape[2:] or offset.size(0) != input.size(0):
        raise RuntimeError(f"{name}: offset must be (B, {ndim}, *spatial) for input (B, C, *spatial)")
    if offset.device != input.device:
        raise RuntimeError("expected all tensors to be on the same CUDA device")
    if input.dtype not in (torch.float32, torch.float16):
        raise RuntimeError(f'"{name}" not implemented for \'{str(input.dtype).replace("torch.", "")}\'')
    if offset.dtype != input.dtype and not (input.dtype == torch.float16 and offset.dtype == torch.float32):
        raise RuntimeError(f"expected scalar type {input.dtype} but found {offset.dtype}")
    assert input.is_contiguous(), "input tensor has to be contiguous"
    offset = offset.contiguous()
    out = torch.empty_like(input)
    _launch(_FN["mvr_apply_offset_%dd" % ndim], input.device,
            (input.data_ptr(), offset.data_ptr(), out.data_ptr(), _DTYPES[input.dtype], _DTYPES[offset.dtype],
             *input.shape, int(order)))
    return out


def _deform(name, ndim, input, weight, bias, offset, geometry, group, deformable_groups, order):
    """The reference's ``deform_2d`` / ``deform_3d`` (medvision/csrc/vision.cpp:76-77) for the one
    configuration its Python layer uses (medvision/ops/cuda_fun_tools.py:94-167): 1x1(x1) kernel,
    stride 1, no padding, dilation 1, one group, one deformable group, identity weight and zero
    bias -- i.e. a displacement-field warp.  ``weight`` and ``bias`` are accepted for signature
    compatibility; anything but that configuration is refused."""
    kernel, stride, padding, dilation = geometry
    if not (all(k == 1 for k in kernel) and all(v == 1 for v in stride) and all(v == 0 for v in padding)
            and all(v == 1 for v in dilation) and group == 1 and deformable_groups == 1):
        raise NotImplementedError(f"{name}: only the 1x1 identity configuration of apply_offset_* is provided")
    if not input.is_cuda:
        raise RuntimeError("Not implemented on the CPU")
    if input.dim() != ndim + 2:
        raise RuntimeError(f"{name}: expected a {ndim + 2}-D input")
    if tuple(weight.shape) != (input.size(1), input.size(1)) + (1,) * ndim:
        raise NotImplementedError(f"{name}: the weight must be the channel identity")
    if offset.dtype != input.dtype:
        # the reference reinterprets with tensor.data<scalar_t>(), which throws on a mismatch
        raise RuntimeError(f"expected scalar type {input.dtype} but found {offset.dtype}")
    return apply_offset(input, offset, order)


def deform_2d(input, weight, bias, offset, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, dilation_h,
              dilation_w, group, deformable_groups, im2col_step, order):
    return _deform("deform_2d", 2, input, weight, bias, offset,
                   ((kernel_h, kernel_w), (stride_h, stride_w), (pad_h, pad_w), (dilation_h, dilation_w)),
                   group, deformable_groups, order)


def deform_3d(input, weight, bias, offset, kernel_d, kernel_h, kernel_w, stride_d, stride_h, stride_w, pad_d, pad_h,
              pad_w, dilation_d, dilation_h, dilation_w, group, deformable_groups, im2col_step, order):
    return _deform("deform_3d", 3, input, weight, bias, offset,
                   ((kernel_d, kernel_h, kernel_w), (stride_d, stride_h, stride_w), (pad_d, pad_h, pad_w),
                    (dilation_d, dilation_h, dilation_w)), group, deformable_groups, order)
