"""TEST INFRASTRUCTURE -- not product code.

ctypes front end of ``oracle/libmvr_oracle.so`` (built from ``oracle/mvr_oracle.cpp`` by
``make -C oracle port``): the CPU restatement of the reference's RoI Align /
RoI Align Rotated / affine kernels on torch CPU tensors.
"""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmvr_oracle.so")
_lib = None

DTYPES = {torch.float32: 0, torch.float16: 1, torch.float64: 2}
KIND_BOX, KIND_ROTATED = 0, 1
ROI_WIDTH = {(2, KIND_BOX): 5, (3, KIND_BOX): 7, (2, KIND_ROTATED): 6, (3, KIND_ROTATED): 10}


def build():
    subprocess.check_call(["make", "-C", _HERE, "port"], stdout=subprocess.DEVNULL)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, i32, f32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p
        L.mvr_oracle_fwd.restype = i32
        L.mvr_oracle_fwd.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i64, i64,
                                     i32, i32, i32, f32, i32, i32, i32, i32, i32, vp]
        L.mvr_oracle_bwd.restype = i32
        L.mvr_oracle_bwd.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i64, i64,
                                     i32, i32, i32, f32, i32, i32, i32, i32, i32, i32, vp]
        L.mvr_oracle_offset.restype = i32
        L.mvr_oracle_offset.argtypes = [vp, vp, vp, i32, i32, i64, i64, i64, i64, i64, i32, i32, i32]
        L.mvr_oracle_max_threads.restype = i32
        _lib = L
    return _lib


def max_threads():
    return lib().mvr_oracle_max_threads()


def _dims(shape, out_size):
    if len(shape) == 4:
        N, C, H, W = shape
        D = 1
        oh, ow = out_size
        od = 1
        ndim = 2
    else:
        N, C, D, H, W = shape
        od, oh, ow = out_size
        ndim = 3
    return ndim, N, C, D, H, W, od, oh, ow


def _trig_ptr(trig, rois, ndim, kind):
    if trig is None:
        return None, None
    assert kind == KIND_ROTATED
    trig = trig.detach().cpu().to(rois.dtype).contiguous()
    assert tuple(trig.shape) == (rois.shape[0], 2 if ndim == 2 else 6)
    return trig, trig.data_ptr()


def device_trig(rois):
    """cos/sin of the rois' angles evaluated with the DEVICE's sinf/cosf (torch CUDA kernels call
    the same functions), in the layout ``trig=`` expects: 2D (R,2) [cos, sin]; 3D (R,6)
    [cos ax, sin ax, cos ay, sin ay, cos az, sin az].  For half rois the argument is widened to
    float and the result rounded to half, as the reference does."""
    ang = rois[:, 5:6] if rois.shape[1] == 6 else rois[:, 7:10]
    a = ang.cuda().float()
    t = torch.stack([torch.cos(a), torch.sin(a)], dim=2).reshape(rois.shape[0], -1)
    return t.to(rois.dtype).cpu()


def forward(features, rois, out_size, kind, spatial_scale=1.0, sampling_ratio=0, aligned=True, order=1,
            fma_mode=0, nthreads=0, trig=None):
    """Reference forward on CPU tensors.  ``kind``: KIND_BOX (RoIAlign) or KIND_ROTATED
    (RoIAlignRotated / affine_*).  Returns (R, C, [od,] oh, ow) in the feature dtype.
    ``trig``: optional table from :func:`device_trig`."""
    features = features.detach().cpu().contiguous()
    rois = rois.detach().cpu().to(features.dtype).contiguous()
    ndim, N, C, D, H, W, od, oh, ow = _dims(tuple(features.shape), tuple(out_size))
    assert rois.dim() == 2 and rois.shape[1] == ROI_WIDTH[(ndim, kind)], "wrong roi size"
    R = rois.shape[0]
    out = torch.empty((R, C) + tuple(out_size), dtype=features.dtype)
    trig, tp = _trig_ptr(trig, rois, ndim, kind)
    rc = lib().mvr_oracle_fwd(features.data_ptr(), rois.data_ptr(), out.data_ptr(), DTYPES[features.dtype],
                              ndim, kind, N, C, D, H, W, R, od, oh, ow, float(spatial_scale),
                              int(sampling_ratio), int(bool(aligned)), int(order), int(fma_mode), int(nthreads), tp)
    if rc < 0:
        raise ValueError(f"mvr_oracle_fwd: bad argument ({rc})")
    if rc == 1:
        raise IndexError("roi batch index outside [0, N)")
    return out


def backward(grad_out, rois, feature_size, kind, spatial_scale=1.0, sampling_ratio=0, aligned=True, order=1,
             fma_mode=0, wide_acc=False, nthreads=0, trig=None):
    """Reference backward: gradient w.r.t. the features, shape ``feature_size``, dtype of grad_out."""
    grad_out = grad_out.detach().cpu().contiguous()
    rois = rois.detach().cpu().to(grad_out.dtype).contiguous()
    out_size = tuple(grad_out.shape[2:])
    ndim, N, C, D, H, W, od, oh, ow = _dims(tuple(feature_size), out_size)
    assert rois.dim() == 2 and rois.shape[1] == ROI_WIDTH[(ndim, kind)], "wrong roi size"
    R = rois.shape[0]
    assert grad_out.shape[0] == R and grad_out.shape[1] == C
    grad_in = torch.zeros(tuple(feature_size), dtype=grad_out.dtype)
    trig, tp = _trig_ptr(trig, rois, ndim, kind)
    rc = lib().mvr_oracle_bwd(grad_out.data_ptr(), rois.data_ptr(), grad_in.data_ptr(), DTYPES[grad_out.dtype],
                              ndim, kind, N, C, D, H, W, R, od, oh, ow, float(spatial_scale),
                              int(sampling_ratio), int(bool(aligned)), int(order), int(fma_mode),
                              int(bool(wide_acc)), int(nthreads), tp)
    if rc < 0:
        raise ValueError(f"mvr_oracle_bwd: bad argument ({rc})")
    if rc == 1:
        raise IndexError("roi batch index outside [0, N)")
    return grad_in


def apply_offset(img, offset, order=1, fma_mode=0, nthreads=0):
    """CPU restatement of ``apply_offset_2d/3d`` (medvision/ops/cuda_fun_tools.py:94-167):
    img (B, C, [D,] H, W), offset (B, ndim, [D,] H, W) in the image's dtype."""
    img = img.detach().cpu().contiguous()
    offset = offset.detach().cpu().to(img.dtype).contiguous()
    ndim = img.dim() - 2
    assert tuple(offset.shape) == (img.shape[0], ndim) + tuple(img.shape[2:])
    B, C = img.shape[:2]
    D = img.shape[2] if ndim == 3 else 1
    H, W = img.shape[-2:]
    out = torch.empty_like(img)
    rc = lib().mvr_oracle_offset(img.data_ptr(), offset.data_ptr(), out.data_ptr(), DTYPES[img.dtype], ndim,
                                 B, C, D, H, W, order, fma_mode, nthreads)
    if rc < 0:
        raise ValueError("mvr_oracle_offset: argument error %d" % rc)
    return out
