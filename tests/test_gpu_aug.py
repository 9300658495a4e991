"""The batched augmentations end to end on the GPU, against the CPU restatement run on the rois
the transform built."""
import numpy as np
import pytest
import torch

from oracle import port
from util import n_mismatch

pytestmark = pytest.mark.gpu


def _result(shape, dtype, seed, seg=True):
    g = torch.Generator().manual_seed(seed)
    img = torch.rand(shape, generator=g).to(dtype).cuda()
    res = {"img_dim": len(shape) - 2, "img": img, "img_fields": ["img"], "seg_fields": []}
    if seg:
        res["gt_seg"] = torch.randint(0, 5, shape, generator=g, dtype=torch.int32).cuda()
        res["seg_fields"] = ["gt_seg"]
    return res


def _check(t, res_in, out_size, sampling_ratio=1):
    img_in, seg_in = res_in["img"].clone(), res_in["gt_seg"].clone()
    res = t(res_in)
    rois = t._rois()
    trig = port.device_trig(rois.to(img_in.dtype))
    want = port.forward(img_in.cpu(), rois, out_size, port.KIND_ROTATED, 1.0, sampling_ratio, True, t.order,
                        trig=trig, fma_mode=0 if img_in.dtype == torch.float16 else REF_FM)
    assert n_mismatch(res["img"], want) == 0
    want_seg = port.forward(seg_in.float().cpu(), rois, out_size, port.KIND_ROTATED, 1.0, 1, True, 0,
                            trig=port.device_trig(rois), fma_mode=REF_FM).int()
    assert res["gt_seg"].dtype == torch.int32
    assert torch.equal(res["gt_seg"].cpu(), want_seg)
    assert res["history"][-1] == t.name and t.key_name in res
    return res


REF_FM = 1 | (1 << 1) | (1 << 2) | (1 << 3) | (1 << 5) | (1 << 7) | (1 << 10) | (1 << 13) | \
    (1 << 16) | (1 << 18) | (2 << 20) | (1 << 22)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_resize(dtype):
    from medvision_b200.aug_cuda_batch import BatchCudaResize
    t = BatchCudaResize(factor=(0.5, 0.75, 0.5), order=1)
    res = _check(t, _result((2, 1, 16, 24, 32), dtype, 1), (8, 18, 16))
    assert res["img"].shape == (2, 1, 8, 18, 16)
    # a factor of one leaves the fields untouched
    r2 = _result((1, 1, 8, 8, 8), dtype, 2)
    before = r2["img"]
    assert BatchCudaResize(factor=(1.0, 1.0, 1.0))(r2)["img"] is before


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_random_affine_3d_and_2d(dtype):
    from medvision_b200.aug_cuda_batch import BatchCudaRandomAffine
    np.random.seed(3)
    t = BatchCudaRandomAffine(1.0, scale=0.2, shift=0.1, rotate=25)
    _check(t, _result((3, 2, 12, 24, 32), dtype, 3), (12, 24, 32))
    t = BatchCudaRandomAffine(1.0, scale=0.2, shift=0.1, rotate=25, sampling_ratio=2)
    res = _result((3, 2, 20, 24), dtype, 4)
    img_in = res["img"].clone()
    out = t(res)
    rois = t._rois()
    want = port.forward(img_in.cpu(), rois, (20, 24), port.KIND_ROTATED, 1.0, 2, True, 1,
                        trig=port.device_trig(rois.to(dtype)), fma_mode=0 if dtype == torch.float16 else REF_FM)
    assert n_mismatch(out["img"], want) == 0


def test_crop_with_affine_times_equals_replicated_batch():
    from medvision_b200.aug_cuda_batch import BatchCudaCropRandomWithAffine
    from medvision_b200.ops import affine_3d
    np.random.seed(5)
    t = BatchCudaCropRandomWithAffine(patch_size=(8, 16, 16), scale=0.1, shift=0, rotate=20, times=3)
    res = _result((2, 1, 20, 40, 48), torch.float16, 5)
    img_in = res["img"].clone()
    out = _check(t, res, (8, 16, 16))
    assert out["img"].shape == (6, 1, 8, 16, 16)
    # the reference's way: concatenate `times` copies and give every copy its own roi
    rois = t._rois()
    rep = torch.cat([img_in] * 3)
    rois_rep = rois.clone()
    rois_rep[:, 0] = torch.arange(6)
    want = affine_3d(rep, rois_rep.cuda(), (8, 16, 16), 1.0, 1, True, 1)
    assert torch.equal(out["img"], want)


def test_host_pipeline_equals_one_call():
    from medvision_b200.ops import affine_3d, affine_from_host
    g = torch.Generator().manual_seed(8)
    vol = torch.rand(3, 2, 12, 24, 32, generator=g).half().pin_memory()
    R = 9
    b = torch.tensor([2, 0, 1, 1, 0, 2, 2, 0, 0]).float().view(-1, 1)  # unsorted batch indices
    rois = torch.cat([b, torch.rand(R, 3, generator=g) * torch.tensor([32., 24., 12.]),
                      torch.rand(R, 3, generator=g) * 10 + 4, torch.zeros(R, 2), torch.rand(R, 1, generator=g) - .5], 1)
    got = affine_from_host(vol, rois, (6, 8, 8), 1.0, 1, True, 1)
    want = affine_3d(vol.cuda(), rois.cuda(), (6, 8, 8), 1.0, 1, True, 1).cpu()
    assert got.is_pinned() and torch.equal(got, want)
    sorted_rois = rois[torch.argsort(rois[:, 0], stable=True)]
    got2 = affine_from_host(vol, sorted_rois, (6, 8, 8), 1.0, 1, True, 0)
    want2 = affine_3d(vol.cuda(), sorted_rois.cuda(), (6, 8, 8), 1.0, 1, True, 0).cpu()
    assert torch.equal(got2, want2)
    # a second call reuses the cached streams and buffers; batch indices outside the batch give zeros, as on
    # the device; order 3 goes through as well
    bad = rois.clone()
    bad[1, 0], bad[6, 0] = -1, 3
    got3 = affine_from_host(vol, bad, (6, 8, 8), 1.0, 1, True, 1)
    want3 = affine_3d(vol.cuda(), bad.cuda(), (6, 8, 8), 1.0, 1, True, 1).cpu()
    assert torch.equal(got3, want3) and torch.count_nonzero(got3[1]) == 0 and torch.count_nonzero(got3[6]) == 0
    from medvision_b200 import _C
    _C.last_status()  # the device-side call above flagged the two indices
    got4 = affine_from_host(vol.float().pin_memory(), rois, (6, 8, 8), 1.0, 1, True, 3)
    want4 = affine_3d(vol.float().cuda(), rois.cuda(), (6, 8, 8), 1.0, 1, True, 3).cpu()
    assert torch.equal(got4, want4)


def test_sliding_window_patches_are_the_slices():
    from medvision_b200.aug_cuda import CudaPatches
    g = torch.Generator().manual_seed(9)
    img = torch.rand(2, 16, 24, 32, generator=g).half().cuda()
    seg = torch.randint(0, 4, (1, 16, 24, 32), generator=g, dtype=torch.int32).cuda()
    res = {"img_dim": 3, "img": img, "gt_seg": seg, "img_fields": ["img"], "seg_fields": ["gt_seg"]}
    t = CudaPatches(patch_size=(8, 8, 16), overlap=0.5)
    res = t(res)
    patches, seg_patches = res["patches_img"], res["patches_gt_seg"]
    assert patches.shape == (len(t.params), 2, 8, 8, 16) and seg_patches.dtype == torch.int32
    for k, (x0, y0, z0, x1, y1, z1) in enumerate(t.params.tolist()):
        assert torch.equal(patches[k], img[:, z0:z1, y0:y1, x0:x1])
        assert torch.equal(seg_patches[k], seg[:, z0:z1, y0:y1, x0:x1])


@pytest.mark.parametrize("shape,dtype", [((2, 2, 16, 24, 32), torch.float16), ((2, 2, 16, 24, 32), torch.float32),
                                         ((3, 1, 40, 48), torch.float32)])
def test_elastic_deformation(shape, dtype):
    """The dense field is one Catmull-Rom affine resample of the coarse field; the image is warped
    linearly, the label with nearest; backward uses the negated field."""
    from medvision_b200.aug_cuda_batch import BatchCudaRandomElasticDeformation
    dim = len(shape) - 2
    np.random.seed(5)
    t = BatchCudaRandomElasticDeformation(1.0, num_control_points=7, max_displacement=0.9)
    res = _result(shape, dtype, 9)
    img_in, seg_in = res["img"].clone(), res["gt_seg"].clone()
    res = t(res)
    coarse = torch.from_numpy(t.params).permute(0, dim + 1, *range(1, dim + 1)).contiguous() / 2
    # roi of the blow-up: centred on the grid, 3 control points narrower (the locked border)
    roi = torch.tensor([[b] + [3.5] * dim + [4.0] * dim + [0.0] * (1 if dim == 2 else 3) for b in range(shape[0])])
    field = port.forward(coarse, roi, shape[2:], port.KIND_ROTATED, 1.0, 1, True, 3, trig=port.device_trig(roi),
                         fma_mode=REF_FM)
    dense = t.dense_field(img_in.device)
    assert dense.dtype == torch.float32 and dense.shape == (shape[0], dim) + tuple(shape[2:])
    torch.testing.assert_close(dense.cpu(), field, rtol=1e-5, atol=1e-6)
    assert float(dense.abs().max()) > 0.5
    # the warp itself, on the field the GPU built
    fm = 0 if dtype == torch.float16 else REF_FM
    assert n_mismatch(res["img"], port.apply_offset(img_in, dense, 1, fma_mode=fm)) == 0
    want_seg = port.apply_offset(seg_in.to(dtype), dense, 0, fma_mode=fm).int()
    assert res["gt_seg"].dtype == torch.int32 and torch.equal(res["gt_seg"].cpu(), want_seg)
    # the inverse pass samples with the negated field
    warped, warped_seg = res["img"].clone(), res["gt_seg"].clone()
    back = t.backward(res)
    assert torch.equal(t.tmp_params, -dense) and t.key_name not in back
    assert n_mismatch(back["img"], port.apply_offset(warped, -dense, 1, fma_mode=fm)) == 0
    assert torch.equal(back["gt_seg"].cpu(), port.apply_offset(warped_seg.to(dtype), -dense, 0, fma_mode=fm).int())


LABEL_CASES = [
    # spatial, out_size, rotation kind
    ((12, 40, 48), (16, 32, 40), "planar"),
    ((12, 40, 48), (16, 32, 40), "general"),
    ((10, 22, 27), (12, 20, 23), "planar"),      # odd width: scalar stores
    ((9, 12, 14), (3, 4, 5), "general"),         # small output: flat kernel
    ((40, 48), (32, 36), "planar"),
]


@pytest.mark.parametrize("spatial,out_size,rot", LABEL_CASES)
@pytest.mark.parametrize("dtype", [torch.uint8, torch.int16, torch.int32, torch.int64])
def test_label_resample_equals_float_nearest_path(spatial, out_size, rot, dtype):
    """affine_label_* on the integer tensor = affine_*(seg.float(), ..., order=0).int(): against the
    restatement, the library's own float path and, when present, the reference's kernels."""
    from medvision_b200.ops import affine_2d, affine_3d, affine_label_2d, affine_label_3d
    from oracle import ref
    ndim = len(spatial)
    g = torch.Generator().manual_seed(hash((spatial, out_size, rot)) % 1000)
    hi = {torch.uint8: 255, torch.int16: 3000, torch.int32: 70000, torch.int64: 1 << 20}[dtype]
    seg = torch.randint(0, hi, (2, 2) + spatial, generator=g).to(dtype)
    R = 5
    b = torch.randint(0, 2, (R, 1), generator=g).float()
    centre = torch.tensor(spatial[::-1], dtype=torch.float32) * (0.3 + 0.4 * torch.rand(R, ndim, generator=g))
    size = torch.tensor(spatial[::-1], dtype=torch.float32) * (0.5 + torch.rand(R, ndim, generator=g))
    if ndim == 2:
        ang = (torch.rand(R, 1, generator=g) - 0.5) * 1.5
    else:
        ang = (torch.rand(R, 3, generator=g) - 0.5) * 1.2
        if rot == "planar":
            ang[:, :2] = 0
    rois = torch.cat([b, centre, size, ang], 1)
    rois[R - 1, 0] = 7  # a batch index outside the batch: zeros
    fn, lab = (affine_2d, affine_label_2d) if ndim == 2 else (affine_3d, affine_label_3d)
    got = lab(seg.cuda(), rois.cuda(), out_size)
    assert got.dtype == torch.int32 and got.shape == (R, 2) + out_size
    good = rois[:R - 1]
    want = port.forward(seg.float(), good, out_size, port.KIND_ROTATED, 1.0, 1, True, 0, trig=port.device_trig(good),
                        fma_mode=REF_FM).int()
    assert torch.equal(got[:R - 1].cpu(), want)
    assert torch.equal(got, fn(seg.cuda().float(), rois.cuda(), out_size, 1.0, 1, True, 0).int())
    assert not bool(got[R - 1].any())
    if ref.available():
        live = ref.forward(seg.cuda().float(), rois[:R - 1].cuda(), out_size, port.KIND_ROTATED, 1.0, 1, True, 0,
                           affine=True).int()
        assert torch.equal(got[:R - 1], live)


def _single(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return {"img_dim": len(shape) - 1, "img": torch.rand(shape, generator=g).to(dtype).cuda(), "img_fields": ["img"],
            "gt_seg": torch.randint(0, 5, shape, generator=g, dtype=torch.int32).cuda(), "seg_fields": ["gt_seg"],
            "img_spacing": (1.0,) * (len(shape) - 1)}


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_single_sample_transforms_equal_the_batched_ones_on_a_batch_of_one(dtype):
    import medvision_b200.aug_cuda as one
    import medvision_b200.aug_cuda_batch as many
    shape = (2, 12, 24, 32)
    pairs = [
        (one.CudaResize(factor=(0.5, 0.75, 0.5)), many.BatchCudaResize(factor=(0.5, 0.75, 0.5))),
        (one.CudaRandomAffine(1.0, 0.2, 0.1, 25), many.BatchCudaRandomAffine(1.0, 0.2, 0.1, 25)),
        (one.CudaRandomRotate(1.0, 40), many.BatchCudaRandomRotate(1.0, 40)),
        (one.CudaCropRandomWithAffine((8, 16, 16), 0.1, 0.05, 20),
         many.BatchCudaCropRandomWithAffine((8, 16, 16), 0.1, 0.05, 20)),
        (one.CudaCropCenterWithAffine((8, 16, 16), 0.1, 0.05, 20),
         many.BatchCudaCropCenterWithAffine((8, 16, 16), 0.1, 0.05, 20)),
        (one.CudaRandomElasticDeformation(1.0, 7, 0.9), many.BatchCudaRandomElasticDeformation(1.0, 7, 0.9)),
    ]
    for k, (a, b) in enumerate(pairs):
        ra = _single(shape, dtype, 30 + k)
        rb = {"img_dim": 3, "img": ra["img"].unsqueeze(0), "img_fields": ["img"],
              "gt_seg": ra["gt_seg"].unsqueeze(0), "seg_fields": ["gt_seg"], "img_spacing": (1.0, 1.0, 1.0)}
        np.random.seed(100 + k)
        ra = a(ra)
        np.random.seed(100 + k)
        rb = b(rb)
        assert torch.equal(ra["img"], rb["img"][0]), a.name
        assert ra["gt_seg"].dtype == torch.int32 and torch.equal(ra["gt_seg"], rb["gt_seg"][0]), a.name
        assert ra["history"] == [a.name]
        if "Elastic" not in a.name:
            assert ra["img_shape"] == tuple(ra["img"].shape)


def test_single_sample_crop_repeats_and_resize_backward():
    import medvision_b200.aug_cuda as one
    res = _single((1, 16, 32, 32), torch.float16, 41)
    np.random.seed(7)
    crops = one.CudaCropRandomWithAffine((8, 16, 16), 0.1, 0.05, 20, times=3)(res)
    assert len(crops) == 3 and all(c["img"].shape == (1, 8, 16, 16) and c["gt_seg"].shape == (1, 8, 16, 16) for c in crops)
    assert not torch.equal(crops[0]["img"], crops[1]["img"])
    assert res["img"].shape == (1, 16, 32, 32)  # the source sample is left as it was
    t = one.CudaResize(factor=(0.5, 0.5, 0.5))
    small = t(_single((1, 16, 32, 32), torch.float32, 42))
    assert small["img"].shape == (1, 8, 16, 16) and small["img_spacing"] == (2.0, 2.0, 2.0)
    back = t(small, forward=False)
    assert back["img"].shape == (1, 16, 32, 32) and back["gt_seg"].shape == (1, 16, 32, 32)
    assert back["history"] == [] and t.key_name not in back


def _graph_node_counts(fn):
    """Capture `fn` into a CUDA graph and count its nodes by kind (kernels, copies)."""
    from cuda.bindings import runtime as rt
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph(keep_graph=True)
    with torch.cuda.stream(side):
        fn()  # lazy set-up (staging buffers, function attributes) outside the capture
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            out = fn()
    torch.cuda.synchronize()
    raw = graph.raw_cuda_graph()
    err, _, n = rt.cudaGraphGetNodes(raw, 0)
    assert err == rt.cudaError_t.cudaSuccess
    err, nodes, n = rt.cudaGraphGetNodes(raw, n)
    kinds = {}
    for node in nodes[:n]:
        err, kind = rt.cudaGraphNodeGetType(node)
        name = getattr(kind, "name", str(kind))
        kinds[name] = kinds.get(name, 0) + 1
    graph.instantiate()
    graph.replay()
    torch.cuda.synchronize()
    return kinds, out


def test_image_and_label_field_cost_the_launches_of_the_image_alone():
    """A 3D RandomAffine on an image field and a label field: one asynchronous roi upload and the two overlapped
    launches a rotated dense forward takes anyway (the label's work rides along with the first) -- no roi cast
    kernel, no label launch, no float copy of the labels; results bit-equal to the separate calls."""
    from medvision_b200.aug_cuda_batch import BatchCudaRandomAffine
    from medvision_b200.ops import affine_3d, affine_label_3d
    np.random.seed(11)
    t = BatchCudaRandomAffine(1.0, scale=0.2, shift=0.1, rotate=25)
    src = _result((2, 1, 32, 48, 64), torch.float16, 5)
    t(dict(src))  # draws the parameters; the captured calls below reuse them
    rois = t._rois()

    def both():
        res = dict(src)
        t.apply_to_img(res)
        return res["img"], res["gt_seg"]

    kinds, (img, seg) = _graph_node_counts(both)
    assert kinds.get("cudaGraphNodeTypeKernel", 0) == 2, kinds
    assert kinds.get("cudaGraphNodeTypeMemcpy", 0) == 1, kinds
    want_img = affine_3d(src["img"], rois.cuda(), (32, 48, 64), 1.0, 1, True, 1)
    want_seg = affine_label_3d(src["gt_seg"], rois.cuda(), (32, 48, 64), 1.0, True)
    assert torch.equal(img, want_img) and torch.equal(seg, want_seg)
