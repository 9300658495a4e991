"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol that
include/mvr.h declares, validates its arguments before touching CUDA, and the Python layer
keeps the reference's argument and error conventions."""
import ctypes
import os
import re

import pytest
import torch

from util import HERE

ROOT = os.path.dirname(HERE)


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mvr.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mvr_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from medvision_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 16
    for n in names:
        assert hasattr(_lib.lib, n), n
    # and the ctypes prototypes cover every entry point that takes tensors
    for n in names:
        assert n in _lib.PROTOTYPES or n in _lib.OTHER_SYMBOLS, n


def test_argument_errors_come_before_any_cuda_call():
    from medvision_b200 import _lib
    L = _lib.lib
    null = ctypes.c_void_p(0)
    ok_ptr = ctypes.c_void_p(16)
    base = dict(dtype=0, ndim=3, kind=1, N=1, C=1, D=4, H=4, W=4, R=1, rw=10, od=2, oh=2, ow=2)

    def call(**kw):
        a = dict(base, **kw)
        return L.mvr_roi_resample_fwd(a.get("feat", ok_ptr), ok_ptr, ok_ptr, a["dtype"], a["ndim"], a["kind"], a["N"],
                                      a["C"], a["D"], a["H"], a["W"], a["R"], a["rw"], a["od"], a["oh"], a["ow"],
                                      1.0, 1, 1, a.get("order", 1), null, null)
    assert call(dtype=7) == -1
    assert call(ndim=4) == -2
    assert call(kind=2) == -3
    assert call(order=3) == -4
    assert call(rw=7) == -7 and "wrong roi size" in _lib.strerror(-7)
    assert call(ndim=2, rw=6, D=4) == -5
    assert call(W=0) == -5
    assert call(feat=null) == -6
    # an empty roi list is a no-op, not an error (and launches nothing)
    assert call(R=0) == 0


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    import importlib
    from medvision_b200 import _lib
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or torch fallback"):
        _lib._load()
    importlib.reload(_lib)


def test_ops_reject_cpu_tensors_like_the_reference():
    from medvision_b200.ops import RoIAlign, RoIAlignRotated, affine_2d, affine_3d
    with pytest.raises(RuntimeError, match="RoIAlign is not implemented on CPU"):
        RoIAlign((2, 2), 1.0)(torch.zeros(1, 1, 4, 4), torch.zeros(1, 5))
    with pytest.raises(RuntimeError, match="RoIAlignRotated is not implemented on CPU"):
        RoIAlignRotated((2, 2, 2), 1.0)(torch.zeros(1, 1, 4, 4, 4), torch.zeros(1, 10))
    with pytest.raises(RuntimeError, match="not implemented on CPU"):
        affine_2d(torch.zeros(1, 1, 4, 4), torch.zeros(1, 6), (2, 2), 1.0)
    with pytest.raises(RuntimeError, match="not implemented on CPU"):
        affine_3d(torch.zeros(1, 1, 4, 4, 4), torch.zeros(1, 10), 2, 1.0)


def test_output_size_conventions():
    from medvision_b200.ops import RoIAlign, RoIAlignRotated, affine_3d
    from medvision_b200.ops.roi_align_nd import roi_align_2d
    from medvision_b200.ops._common import parse_output_size
    assert parse_output_size(3, 3) == (3, 3, 3)
    assert parse_output_size((1, 2), 2) == (1, 2)
    with pytest.raises(TypeError, match="must be an integer or tuple of integers"):
        roi_align_2d(torch.zeros(1, 1, 4, 4), torch.zeros(1, 5), [2, 2], 1.0)
    with pytest.raises(AssertionError):
        parse_output_size((1, 2, 3), 2)
    with pytest.raises(Exception, match="incorrect output size"):
        RoIAlign((2,), 1.0)
    with pytest.raises(Exception, match="incorrect output size"):
        RoIAlignRotated((2, 2, 2, 2), 1.0)
    with pytest.raises(AssertionError, match="only support order"):
        RoIAlign((2, 2), 1.0)(torch.zeros(1, 1, 4, 4), torch.zeros(1, 5), order=3)
    with pytest.raises(RuntimeError, match="not implemented on CPU"):
        affine_3d(torch.zeros(1, 1, 4, 4, 4), torch.zeros(1, 10), 2, 1.0, order=3)  # order 3 is accepted
    with pytest.raises(AssertionError, match="not supported"):
        affine_3d(torch.zeros(1, 1, 4, 4, 4), torch.zeros(1, 10), 2, 1.0, order=2)
    with pytest.raises(AssertionError, match="float16 or float32"):
        affine_3d(torch.zeros(1, 1, 4, 4, 4, dtype=torch.float64), torch.zeros(1, 10), 2, 1.0)
    m = RoIAlignRotated((2, 3), 0.5, sampling_ratio=2, aligned=False)
    assert (m.dim, m.spatial_scale, m.sampling_ratio, m.aligned) == (2, 0.5, 2, False)


def test_build_is_sm_100a_only_and_has_no_fallback_sources():
    """setup.py / medvision_b200.build: one nvcc call for sm_100a, nothing else (no other architecture, no
    curand, no Triton, no CPU implementation to fall back to)."""
    import os
    from medvision_b200 import build
    flags = " ".join(build.NVCC_FLAGS)
    assert "arch=compute_100a,code=sm_100a" in flags
    assert flags.count("-gencode") == 1 and "curand" not in flags
    root = os.path.dirname(os.path.dirname(os.path.abspath(build.__file__)))
    setup_py = open(os.path.join(root, "setup.py")).read()
    assert "medvision_b200" in setup_py and "build_py" in setup_py and "triton" not in setup_py.lower().replace("no triton", "")
    for dirpath, _, files in os.walk(os.path.join(root, "medvision_b200")):
        for f in files:
            if f.endswith(".py"):
                src = open(os.path.join(dirpath, f)).read()
                assert "import triton" not in src and "torch.compile" not in src, f
