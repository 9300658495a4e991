"""Host logic of the batched augmentations (no GPU): parameter draws and roi construction follow
medvision/aug_cuda_batch/aug_spatial.py."""
import math
import random

import numpy as np
import pytest
import torch

from medvision_b200.aug_cuda_batch import (BatchCudaCropCenterWithAffine, BatchCudaCropRandomWithAffine,
                                           BatchCudaRandomAffine, BatchCudaRandomElasticDeformation, BatchCudaRandomRotate,
                                           BatchCudaRandomScale,
                                           BatchCudaRandomShift, BatchCudaResize)


def _result(shape=(3, 1, 8, 10, 12)):
    return {"img_dim": len(shape) - 2, "img": torch.zeros(shape), "img_fields": ["img"], "seg_fields": []}


def test_resize_roi_is_the_whole_image():
    t = BatchCudaResize(factor=(0.5, 0.5, 0.25))
    res = _result()
    t._forward_params(res)
    rois = t._rois()
    assert rois.shape == (3, 10)
    assert rois[:, 0].tolist() == [0, 1, 2]
    # xyz order: centre = shape / 2, size = shape, no rotation
    assert torch.equal(rois[0, 1:], torch.tensor([6., 5., 4., 12., 10., 8., 0., 0., 0.]))
    assert res["BatchCudaResize_params"] == (0.5, 0.5, 0.25)
    t2 = BatchCudaResize(scale=(4, -1, 6))
    t2._forward_params(_result())
    assert t2.params == (0.5, 1.0, 0.5)
    t2._backward_params({"img_dim": 3, "img": torch.zeros(3, 1, 4, 10, 6), "BatchCudaResize_params": t2.params})
    assert t2.params == (2.0, 1.0, 2.0)


def test_random_affine_draws_and_roi_formula():
    np.random.seed(7)
    t = BatchCudaRandomAffine(1.0, scale=0.2, shift=0.1, rotate=30)
    res = _result()
    t._forward_params(res)
    # the same draws, in the reference's order: per sample scale, dim shifts, rotation
    np.random.seed(7)
    for b in range(3):
        sc = 1 + np.random.uniform(-0.2, 0.2)
        sh = [np.random.uniform(-0.1, 0.1) for _ in range(3)]
        ro = math.pi * np.random.uniform(-30, 30) / 180
        assert np.allclose(t.params["scales"][b], [sc] * 3)
        assert np.allclose(t.params["shifts"][b], sh)
        assert np.allclose(t.params["rotate"][b], [ro])
    rois = t._rois()
    shape = np.array([12., 10., 8.], dtype=np.float32)
    for b in range(3):
        sc = t.params["scales"][b].astype(np.float32)
        sh = t.params["shifts"][b].astype(np.float32)
        want_c = shape / 2 - shape * sh / sc
        want_s = shape / sc
        assert np.array_equal(rois[b, 1:4].numpy(), want_c.astype(np.float32))
        assert np.array_equal(rois[b, 4:7].numpy(), want_s.astype(np.float32))
        assert rois[b, 7] == 0 and rois[b, 8] == 0  # rotation about z only
        assert rois[b, 9] == np.float32(t.params["rotate"][b, 0])
    # inverse parameters
    t._backward_params(res)
    assert np.allclose(t.params["scales"], 1 / res["BatchCudaRandomAffine_params"]["scales"])


def test_single_purpose_subclasses():
    np.random.seed(1)
    t = BatchCudaRandomShift(1.0, shift=0.2)
    t._forward_params(_result())
    assert np.all(t.params["scales"] == 1) and np.all(t.params["rotate"] == 0)
    t = BatchCudaRandomScale(1.0, scale=0.2)
    t._forward_params(_result())
    assert np.all(t.params["shifts"] == 0) and np.all(t.params["rotate"] == 0)
    t = BatchCudaRandomRotate(1.0, rotate=10)
    t._forward_params(_result((2, 1, 9, 9)))
    assert t._rois().shape == (2, 6)


def test_probability_gate_uses_random_random():
    random.seed(3)
    t = BatchCudaRandomRotate(0.0001, rotate=10)
    res = _result()
    t._forward(t._pre_forward(res))  # almost surely skipped: nothing is applied, no params stored
    assert "BatchCudaRandomRotate_params" not in res


def test_crop_times_share_the_images():
    np.random.seed(11)
    t = BatchCudaCropRandomWithAffine(patch_size=(4, 6, 6), scale=0.1, shift=0, rotate=20, times=4)
    res = _result()
    t._forward_params(res)
    rois = t._rois()
    assert rois.shape == (12, 10)
    # patch r*B + b comes from image b: what concatenating `times` copies of the batch would give
    assert rois[:, 0].tolist() == [0, 1, 2] * 4
    start, end = t.params["start"], t.params["end"]
    assert np.all(end - start == np.array([6, 6, 4]))  # xyz
    assert np.all(start >= 0) and np.all(end <= np.array([12, 10, 8]))
    sc = torch.FloatTensor(t.params["scales"])
    assert torch.equal(rois[:, 4:7], torch.FloatTensor(end - start) / sc)
    t = BatchCudaCropCenterWithAffine(patch_size=(4, 6, 6), scale=0, shift=0, rotate=0)
    t._forward_params(_result())
    assert np.all(t.params["start"] == np.array([3, 2, 2]))
    with pytest.raises(AssertionError):
        BatchCudaCropRandomWithAffine(patch_size=(40, 6, 6), scale=0, shift=0, rotate=0)._forward_params(_result())


def test_sliding_window_anchors():
    from medvision_b200.aug_cuda import CudaPatches
    t = CudaPatches(patch_size=(8, 8, 8), overlap=0.5)
    res = {"img_dim": 3, "img": torch.zeros(1, 16, 20, 24)}
    t._forward_params(res)
    # stride 4; grid counts max((s-1)//4, 1) = 3, 4, 5 along z, y, x; x fastest; boxes in xyz order
    assert t.params.shape == (60, 6)
    assert t.params[0].tolist() == [0, 0, 0, 8, 8, 8] and t.params[1].tolist() == [4, 0, 0, 12, 8, 8]
    assert t.params[-1].tolist() == [16, 12, 8, 24, 20, 16]
    rois = t._rois()
    assert rois[1].tolist() == [0, 8, 4, 4, 8, 8, 8, 0, 0, 0]
    t2 = CudaPatches(patch_size=(6, 6), overlap=0.0)
    t2._forward_params({"img_dim": 2, "img": torch.zeros(3, 5, 13)})
    assert t2.params.tolist() == [[0, 0, 6, 6], [6, 0, 12, 6]]


@pytest.mark.parametrize("shape,points", [((2, 1, 16, 24, 32), 8), ((2, 1, 24, 32), (6, 7))])
def test_elastic_coarse_field_draws_and_locked_borders(shape, points):
    """Same draws as the reference (one np.random.rand(*grid, dim) per sample), scaled per axis
    to max_displacement half grid cells, two outermost control points of every axis zeroed."""
    dim = len(shape) - 2
    t = BatchCudaRandomElasticDeformation(1.0, num_control_points=points, max_displacement=0.8)
    np.random.seed(11)
    res = _result(shape)
    t._forward_params(res)
    grid = t.to_tuple(points, dim)
    assert t.params.shape == (2,) + grid + (dim,) and t.params.dtype == np.float32
    np.random.seed(11)
    for b in range(2):
        draw = 2 * np.random.rand(*grid, dim).astype(np.float32) - 1
        for d in range(dim):
            reach = 0.8 * (shape[2 + d] / (grid[d] - 1)) / 2
            inner = (slice(2, -2),) * dim
            np.testing.assert_allclose(t.params[b][inner + (d,)], draw[inner + (d,)] * reach, rtol=1e-6)
            assert np.abs(t.params[b][..., d]).max() <= reach
    for axis in range(dim):
        for pos in (0, 1, -1, -2):
            assert not np.take(t.params, pos, axis=1 + axis).any()
    assert res[t.key_name] is t.params
    # backward negates the stored field and forgets the cached dense field
    t.tmp_params = "stale"
    t._backward_params(res)
    assert t.tmp_params is None and t.key_name not in res
    assert t.canBackward


# ----------------------------------------------------------------------------- single-sample classes
def _sample(shape=(1, 8, 10, 12)):
    return {"img_dim": len(shape) - 1, "img": torch.zeros(shape), "img_fields": ["img"], "seg_fields": [],
            "img_spacing": (1.0,) * (len(shape) - 1)}


def test_single_sample_transforms_draw_like_their_batched_twins():
    """One sample = a batch of one: same draws from numpy's generator, same roi."""
    from medvision_b200.aug_cuda import (CudaCropCenterWithAffine, CudaCropRandomWithAffine, CudaRandomAffine,
                                         CudaResize)
    np.random.seed(4)
    single = CudaRandomAffine(1.0, scale=0.2, shift=0.1, rotate=30)
    single._forward_params(_sample())
    np.random.seed(4)
    batched = BatchCudaRandomAffine(1.0, scale=0.2, shift=0.1, rotate=30)
    batched._forward_params(_result((1, 1, 8, 10, 12)))
    assert torch.equal(single._rois(), batched._rois())
    assert set(single.params) == {"_scales", "_shifts", "_rotate"} and len(single.params["_shifts"]) == 3

    np.random.seed(5)
    crop = CudaCropRandomWithAffine(patch_size=(4, 6, 6), scale=0.1, shift=0.05, rotate=15)
    crop._forward_params(_sample())
    np.random.seed(5)
    bcrop = BatchCudaCropRandomWithAffine(patch_size=(4, 6, 6), scale=0.1, shift=0.05, rotate=15)
    bcrop._forward_params(_result((1, 1, 8, 10, 12)))
    assert torch.allclose(crop._rois(), bcrop._rois())
    start, end = crop.params["start"], crop.params["end"]  # xyz
    assert all(e - s == p for s, e, p in zip(start, end, (6, 6, 4)))

    centre = CudaCropCenterWithAffine(patch_size=(4, 6, 6), scale=0, shift=0, rotate=0)
    centre._forward_params(_sample())
    assert centre.params["start"] == (3, 2, 2) and centre.params["end"] == (9, 8, 6)
    assert torch.equal(centre._rois(), torch.tensor([[0, 6., 5., 4., 6., 6., 4., 0., 0., 0.]]))

    resize = CudaResize(factor=(0.5, 0.5, 0.25))
    resize._forward_params(_sample())
    assert torch.equal(resize._rois(), torch.tensor([[0, 6., 5., 4., 12., 10., 8., 0., 0., 0.]]))


def test_crop_around_the_first_detection_box():
    from medvision_b200.aug_cuda import CudaCropFirstDetWithAffine
    t = CudaCropFirstDetWithAffine(border=1, patch_size=(4, 6, 6), scale=0, shift=0, rotate=0)
    res = _sample()
    res["gt_det"] = torch.tensor([[7., 5., 3., 9., 7., 5., 1., 1.]])  # x1 y1 z1 x2 y2 z2 label score
    for seed in range(20):
        np.random.seed(seed)
        t._forward_params(res)
        (sx, sy, sz), (ex, ey, ez) = t.params["start"], t.params["end"]
        assert (ex - sx, ey - sy, ez - sz) == (6, 6, 4)
        # the box plus its border stays inside the patch wherever the image leaves room
        assert sx <= 6 and ex >= 10 and sy <= 4 and ey >= 8 and sz <= 2 + 1 and ez >= 6 - 1
        assert 0 <= sx and ex <= 12 and 0 <= sy and ey <= 10 and 0 <= sz and ez <= 8
    res["gt_det"] = torch.zeros(0, 8)
    t._forward_params(res)  # no box: a random crop


def test_repeats_make_a_list_of_results_without_copying_tensors():
    from medvision_b200.aug_cuda import CudaAugBase

    class Tag(CudaAugBase):
        def __init__(self):
            super().__init__()
            self.always = True

        @property
        def repeats(self):
            return 3

        def _forward_params(self, result):
            result[self.key_name] = np.random.rand()

    res = _sample()
    out = Tag()(res)
    assert isinstance(out, list) and len(out) == 3
    assert all(o["img"] is res["img"] for o in out)
    assert len({o["Tag_params"] for o in out}) == 3
    assert all(o["history"] == ["Tag"] for o in out) and "history" not in res
