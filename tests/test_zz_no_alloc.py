"""The backward entry point that allocates nothing (mvr_roi_resample_bwd_noalloc).

Some hosts of this library cannot allocate device memory at call time -- a plug-in hook that may
not allocate after initialisation, a worker beside a framework that has reserved the whole GPU
for its own allocator -- so the half-precision dense 3D backward, which normally borrows a
float accumulator volume from the memory pool, also exists with that accumulator in a fixed
array inside the library.  This file checks, through the C ABI, that the variant gives what the
regular entry point gives, twice in a row (the array is shared and keeps old contents between
calls), and that it refuses volumes beyond its fixed capacity.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, grad, rois, gin, stream=None):
    from medvision_b200 import _lib
    N, C, D, H, W = gin.shape
    R = rois.size(0)
    od, oh, ow = grad.shape[2:]
    code = {torch.float16: _lib.MVR_F16, torch.float32: _lib.MVR_F32}[grad.dtype]
    st = torch.cuda.current_stream().cuda_stream if stream is None else stream
    return fn(grad.data_ptr(), rois.data_ptr(), gin.data_ptr(), code, 3, _lib.MVR_ROI_ROTATED, N, C, D, H, W, R,
              rois.size(1), od, oh, ow, 1.0, 1, 1, 1, None, st)


def _job(seed, shape=(2, 2, 24, 40, 48), out=(20, 32, 40), R=5):
    g = torch.Generator().manual_seed(seed)
    N, C, D, H, W = shape
    b = torch.randint(0, N, (R, 1), generator=g).float()
    ext = torch.tensor([W, H, D], dtype=torch.float32)
    centre = ext / 2 + (torch.rand(R, 3, generator=g) - 0.5) * ext * 0.4
    size = ext * (0.6 + 0.6 * torch.rand(R, 3, generator=g))
    ang = (torch.rand(R, 3, generator=g) - 0.5) * 0.8
    ang[0] = 0
    ang[1, :2] = 0
    rois = torch.cat([b, centre, size, ang], 1).half().cuda()
    grad = torch.randn((R, C) + out, generator=g).half().cuda()
    return grad, rois, shape


def test_noalloc_backward_equals_regular_backward_twice_in_a_row():
    from medvision_b200 import _lib
    L = _lib.lib
    for rep, seed in enumerate((101, 202)):  # second call: the shared array still holds call one
        grad, rois, shape = _job(seed)
        want = torch.zeros(shape, dtype=torch.float16, device="cuda")
        got = torch.zeros(shape, dtype=torch.float16, device="cuda")
        assert _call(L.mvr_roi_resample_bwd, grad, rois, want) == 0
        assert _call(L.mvr_roi_resample_bwd_noalloc, grad, rois, got) == 0
        torch.cuda.synchronize()
        assert float(want.abs().max()) > 0
        # Both sum the same half products in a float accumulator; only the order in which the
        # reductions land differs, so the tolerance is that of float summation, far below a half ulp.
        err = (got.float() - want.float()).abs()
        bound = 2e-3 * (want.float().abs() + float(want.float().pow(2).mean().sqrt()))
        assert bool((err <= bound).all()), "call %d: max abs err %g" % (rep, float(err.max()))


def test_noalloc_backward_serves_the_shapes_without_accumulator_too():
    from medvision_b200 import _lib
    L = _lib.lib
    grad, rois, shape = _job(303)
    want = torch.zeros(shape, dtype=torch.float32, device="cuda")
    got = torch.zeros(shape, dtype=torch.float32, device="cuda")
    assert _call(L.mvr_roi_resample_bwd, grad.float(), rois.float(), want) == 0
    assert _call(L.mvr_roi_resample_bwd_noalloc, grad.float(), rois.float(), got) == 0
    torch.cuda.synchronize()
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)


def test_noalloc_backward_refuses_volumes_beyond_its_capacity():
    from medvision_b200 import _lib
    L = _lib.lib
    shape = (1, 1, 129, 256, 128)  # 4 227 072 elements > 4 194 304
    grad, rois, _ = _job(404, shape=shape, out=(16, 32, 32), R=2)
    gin = torch.zeros(shape, dtype=torch.float16, device="cuda")
    rc = _call(L.mvr_roi_resample_bwd_noalloc, grad, rois, gin)
    assert rc == -11
    assert "4194304" in _lib.strerror(rc)
    torch.cuda.synchronize()
    assert float(gin.abs().max()) == 0.0  # nothing was launched
    # the regular entry point takes the same call
    assert _call(L.mvr_roi_resample_bwd, grad, rois, gin) == 0
    torch.cuda.synchronize()


def _pool_high_water(reset=False):
    """High-water mark of the device's default stream-ordered memory pool (which the library must leave alone)."""
    from cuda.bindings import runtime as rt
    dev = torch.cuda.current_device()
    err, pool = rt.cudaDeviceGetDefaultMemPool(dev)
    assert err == rt.cudaError_t.cudaSuccess
    if reset:
        from cuda.bindings.driver import cuuint64_t
        (err,) = rt.cudaMemPoolSetAttribute(pool, rt.cudaMemPoolAttr.cudaMemPoolAttrUsedMemHigh, cuuint64_t(0))
        assert err == rt.cudaError_t.cudaSuccess
    err, used = rt.cudaMemPoolGetAttribute(pool, rt.cudaMemPoolAttr.cudaMemPoolAttrUsedMemHigh)
    assert err == rt.cudaError_t.cudaSuccess
    return int(used)


def test_noalloc_backward_takes_nothing_from_any_memory_pool():
    """The regular half backward borrows its accumulator from the library's own memory pool; the variant must leave
    that pool and the device's default pool where they were."""
    from medvision_b200 import _C, _lib
    L = _lib.lib
    grad, rois, shape = _job(505)
    gin = torch.zeros(shape, dtype=torch.float16, device="cuda")
    assert _call(L.mvr_roi_resample_bwd_noalloc, grad, rois, gin) == 0  # first call: address look-up done
    torch.cuda.synchronize()
    _C.release_cached_memory()
    assert _C.cached_memory_bytes() == 0
    before = _pool_high_water(reset=True)
    assert _call(L.mvr_roi_resample_bwd_noalloc, grad, rois, gin) == 0
    torch.cuda.synchronize()
    assert _pool_high_water() == before and _C.cached_memory_bytes() == 0
    # ... whereas the regular entry point does borrow (the check above can see an allocation): from the library's
    # pool, which keeps the memory for the next call, and not from the device's default pool
    assert _call(L.mvr_roi_resample_bwd, grad, rois, gin) == 0
    torch.cuda.synchronize()
    n = 1
    for s in shape:
        n *= s
    assert _C.cached_memory_bytes() >= 4 * n
    assert _pool_high_water() == before
    _C.release_cached_memory()
    assert _C.cached_memory_bytes() == 0


@pytest.mark.parametrize("case", ["head3d_ratio2", "plane2d"])
def test_noalloc_backward_equals_regular_backward_on_shapes_outside_the_dense_path(case):
    """Detection-head and 2D shapes need no accumulator volume; both entry points send them to the same kernels
    (element-type atomics), so the results agree to the order of the atomics."""
    from medvision_b200 import _lib
    L = _lib.lib
    g = torch.Generator().manual_seed(606)
    if case == "head3d_ratio2":
        shape, out, R, width, nd, ratio = (2, 3, 16, 20, 24), (5, 6, 7), 9, 10, 3, 2
        ext = torch.tensor([24., 20., 16.])
    else:
        shape, out, R, width, nd, ratio = (2, 3, 1, 40, 48), (1, 9, 11), 7, 6, 2, 1
        ext = torch.tensor([48., 40.])
    b = torch.randint(0, 2, (R, 1), generator=g).float()
    centre = ext / 2 + (torch.rand(R, nd, generator=g) - 0.5) * ext * 0.4
    size = ext * (0.3 + 0.5 * torch.rand(R, nd, generator=g))
    ang = (torch.rand(R, 1 if nd == 2 else 3, generator=g) - 0.5) * 0.8
    rois = torch.cat([b, centre, size, ang], 1).cuda()
    grad = torch.randn((R, shape[1]) + out, generator=g).cuda()
    N, C, D, H, W = shape

    def run(fn):
        gin = torch.zeros(shape, device="cuda")
        rc = fn(grad.data_ptr(), rois.data_ptr(), gin.data_ptr(), _lib.MVR_F32, nd, _lib.MVR_ROI_ROTATED, N, C, D, H, W,
                R, width, *out, 1.0, ratio, 1, 1, None, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        return gin

    want, got = run(L.mvr_roi_resample_bwd), run(L.mvr_roi_resample_bwd_noalloc)
    assert float(want.abs().max()) > 0
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
