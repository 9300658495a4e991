"""Seeded inputs of the golden cases (shared by the generator and the tests)."""
import math

import torch

KIND_BOX, KIND_ROTATED = 0, 1


def make_rois(gen, ndim, kind, n_batch, spatial, R, dtype):
    """R rois over a volume of ``spatial`` = (D,H,W) or (H,W): inside, straddling the border,
    fully outside, tiny and large ones.  xyz order, as the reference's layout."""
    ext = torch.tensor(list(reversed(spatial)), dtype=torch.float64)  # (W,H[,D])
    b = torch.randint(0, n_batch, (R, 1), generator=gen).double()
    centre = (torch.rand(R, ndim, generator=gen, dtype=torch.float64) * 1.4 - 0.2) * ext
    size = (torch.rand(R, ndim, generator=gen, dtype=torch.float64) * 0.9 + 0.02) * ext
    size[0] = 0.3            # smaller than one voxel
    centre[1] = ext * 2.5    # entirely outside
    if R > 2:
        size[2] = ext * 1.5  # larger than the volume
    if kind == KIND_BOX:
        rois = torch.cat([b, centre - size / 2, centre + size / 2], 1)
        if R > 3:
            rois[3, 1 + ndim:] = rois[3, 1:1 + ndim] - 1.0  # end < start: size clamps to 1
    else:
        nang = 1 if ndim == 2 else 3
        ang = (torch.rand(R, nang, generator=gen, dtype=torch.float64) * 2 - 1) * math.pi
        ang[0] = 0.0
        if ndim == 3 and R > 4:
            ang[4, :2] = 0.0  # rotation about z only, as the augmentations use it
        rois = torch.cat([b, centre, size, ang], 1)
        if R > 3:
            rois[3, 1 + ndim:1 + 2 * ndim] = 0.0  # zero-size roi
    return rois.to(dtype)


def all_cases():
    """(name, dict) for every golden case."""
    out = []
    seed = 100
    for ndim in (2, 3):
        spatial = (20, 24) if ndim == 2 else (9, 12, 14)
        out_size = (5, 4) if ndim == 2 else (3, 4, 5)
        for kind in (KIND_BOX, KIND_ROTATED):
            for dtype in (torch.float32, torch.float16):
                for order, sr in ((1, 2), (1, 0), (0, 1), (1, 1)):
                    for aligned in ((True, False) if kind == KIND_ROTATED and order == 1 and sr == 2 else (True,)):
                        seed += 1
                        name = "%dd_%s_%s_o%d_s%d_%s" % (
                            ndim, "box" if kind == KIND_BOX else "rot",
                            "f32" if dtype == torch.float32 else "f16", order, sr, "al" if aligned else "na")
                        out.append((name, dict(ndim=ndim, kind=kind, dtype=dtype, order=order, sampling_ratio=sr,
                                               aligned=aligned, spatial=spatial, out_size=out_size, seed=seed,
                                               N=2, C=3, R=7,
                                               spatial_scale={(1, 2): 1.0, (1, 0): 0.5, (0, 1): 0.77, (1, 1): 0.3}[(order, sr)])))
    # Catmull-Rom (order 3) exists in the forward-only affine_2d / affine_3d entry points
    for ndim in (2, 3):
        spatial = (20, 24) if ndim == 2 else (9, 12, 14)
        out_size = (7, 6) if ndim == 2 else (4, 5, 6)
        for dtype in (torch.float32, torch.float16):
            for sr in (1, 2):
                seed += 1
                name = "%dd_affine_%s_o3_s%d" % (ndim, "f32" if dtype == torch.float32 else "f16", sr)
                out.append((name, dict(ndim=ndim, kind=KIND_ROTATED, dtype=dtype, order=3, sampling_ratio=sr,
                                       aligned=True, spatial=spatial, out_size=out_size, seed=seed, N=2, C=3, R=7,
                                       spatial_scale=1.0, affine_only=True)))
    return out


def make_inputs(case):
    gen = torch.Generator().manual_seed(case["seed"])
    dtype = case["dtype"]
    feat = torch.rand((case["N"], case["C"]) + tuple(case["spatial"]), generator=gen, dtype=torch.float64)
    feat = (feat * 2 - 0.5).to(dtype)
    scale = case["spatial_scale"]
    rois = make_rois(gen, case["ndim"], case["kind"], case["N"], case["spatial"], case["R"], torch.float64)
    rois[:, 1:1 + 2 * case["ndim"]] /= scale
    rois = rois.to(dtype)
    grad = torch.randn((case["R"], case["C"]) + tuple(case["out_size"]), generator=gen, dtype=torch.float64).to(dtype)
    return feat, rois, grad


def offset_cases():
    """(name, dict) for the displacement-field warp (apply_offset_2d/3d) golden cases."""
    out = []
    seed = 500
    for ndim in (2, 3):
        for spatial in (((20, 24), (7, 13)) if ndim == 2 else ((9, 12, 14), (5, 6, 7))):
            for dtype in (torch.float32, torch.float16):
                for order in (0, 1, 3):
                    seed += 1
                    name = "offset_%dd_%s_%s_o%d" % (ndim, "x".join(map(str, spatial)),
                                                     "f32" if dtype == torch.float32 else "f16", order)
                    out.append((name, dict(ndim=ndim, dtype=dtype, order=order, spatial=spatial, seed=seed, B=2, C=3)))
    return out


def make_offset_inputs(case):
    """Image in [-0.5, 1.5); field = gaussian displacements (sigma 2.5 voxels, so a good share of
    the samples leaves the image), with a sprinkling of whole-voxel displacements and of samples
    placed exactly on the borders -1, 0, size-1 and size of the validity test."""
    gen = torch.Generator().manual_seed(case["seed"])
    spatial = tuple(case["spatial"])
    ndim = case["ndim"]
    img = (torch.rand((case["B"], case["C"]) + spatial, generator=gen, dtype=torch.float64) * 2 - 0.5)
    off = torch.randn((case["B"], ndim) + spatial, generator=gen, dtype=torch.float64) * 2.5
    pick = torch.rand(off.shape, generator=gen)
    off = torch.where(pick < 0.1, off.round(), off)
    grid = torch.stack(torch.meshgrid(*[torch.arange(n, dtype=torch.float64) for n in spatial], indexing="ij"))[None]
    sizes = torch.tensor(spatial, dtype=torch.float64).reshape((1, ndim) + (1,) * ndim)
    for k, target in enumerate((-1.0 + 0 * sizes, 0 * sizes, sizes - 1, sizes)):
        sel = (pick >= 0.1 + 0.02 * k) & (pick < 0.12 + 0.02 * k)
        off = torch.where(sel, target - grid, off)
    return img.to(case["dtype"]), off.to(case["dtype"])
