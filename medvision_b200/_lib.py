"""ctypes binding of libmvr.so (the C ABI of include/mvr.h).

The library is the only implementation: if it is missing or cannot be loaded, importing
this module raises -- nothing falls back to torch or to the CPU.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmvr.so")

MVR_F32, MVR_F16, MVR_F64 = 0, 1, 2
MVR_ROI_BOX, MVR_ROI_ROTATED = 0, 1
MVR_ERR_ROI_WIDTH = -7
MVR_ERR_UNSUPPORTED = -13
MVR_STATUS_BAD_BATCH_INDEX = 1
MVR_STATUS_TMA_TIMEOUT = 2

_i64, _i32, _f32, _vp = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p

# name -> argtypes, exactly the prototypes of include/mvr.h
_GENERAL = [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _i64, _i64, _i32,
            _i32, _i32, _i32, _f32, _i32, _i32, _i32, _vp, _vp]
_BOX2D = [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _f32, _i32, _i32, _vp, _vp]
_BOX3D = [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _f32, _i32, _i32, _vp, _vp]
_ROT2D = [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _f32, _i32, _i32, _i32, _vp, _vp]
_ROT3D = [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _f32, _i32, _i32, _i32,
          _vp, _vp]

PROTOTYPES = {
    "mvr_roi_resample_fwd": _GENERAL,
    "mvr_roi_resample_bwd": _GENERAL,
    "mvr_roi_resample_bwd_noalloc": _GENERAL,
    "mvr_roi_resample_touched": [_vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _i64, _i64, _i32,
                                 _i32, _i32, _i32, _f32, _i32, _i32, _i32, _vp],
    "mvr_roi_align_2d_forward": _BOX2D,
    "mvr_roi_align_2d_backward": _BOX2D,
    "mvr_roi_align_3d_forward": _BOX3D,
    "mvr_roi_align_3d_backward": _BOX3D,
    "mvr_roi_align_rotated_2d_forward": _ROT2D,
    "mvr_roi_align_rotated_2d_backward": _ROT2D,
    "mvr_roi_align_rotated_3d_forward": _ROT3D,
    "mvr_roi_align_rotated_3d_backward": _ROT3D,
    "mvr_apply_offset_2d": [_vp, _vp, _vp, _i32, _i32, _i64, _i64, _i64, _i64, _i32, _vp],
    "mvr_apply_offset_3d": [_vp, _vp, _vp, _i32, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp],
    "mvr_affine_label_2d": [_vp, _i32, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _f32, _i32, _vp, _vp],
    "mvr_affine_label_3d": [_vp, _i32, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _f32,
                            _i32, _vp, _vp],
    "mvr_affine_fields_3d": [_vp, _i32, _vp, _vp, _i64, _vp, _i32, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32,
                             _i32, _i32, _i32, _f32, _i32, _i32, _vp, _vp],
    "mvr_affine_2d": _ROT2D,
    "mvr_affine_3d": _ROT3D,
}
OTHER_SYMBOLS = ["mvr_strerror", "mvr_version", "mvr_set_float_contraction", "mvr_get_float_contraction",
                 "mvr_selftest_tma_skip_plane", "mvr_cached_memory_bytes", "mvr_release_cached_memory"]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m medvision_b200.build` "
            "(medvision_b200 has no CPU or torch fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = _i32
        fn.argtypes = argtypes
    lib.mvr_strerror.restype = ctypes.c_char_p
    lib.mvr_strerror.argtypes = [_i32]
    lib.mvr_version.restype = _i32
    lib.mvr_set_float_contraction.restype = _i32
    lib.mvr_set_float_contraction.argtypes = [_i32]
    lib.mvr_get_float_contraction.restype = _i32
    lib.mvr_selftest_tma_skip_plane.restype = _i32
    lib.mvr_cached_memory_bytes.restype = ctypes.c_longlong
    lib.mvr_cached_memory_bytes.argtypes = []
    lib.mvr_release_cached_memory.restype = _i32
    lib.mvr_release_cached_memory.argtypes = []
    lib.mvr_selftest_tma_skip_plane.argtypes = [_i32]
    return lib


lib = _load()


def strerror(code):
    return lib.mvr_strerror(code).decode()
