"""TEST / MEASUREMENT INFRASTRUCTURE -- not product code.

Restatement of the reference's torch-function RoIAlign
(medvision/ops/pytorch_ops/roi_align.py:9-105): a Python loop over the rois, each one an
``affine_grid`` + ``grid_sample(align_corners=False)`` on the roi's sample.  It is the CPU timing
baseline "the reference's torch-function path"; it is NOT a parity oracle for the CUDA op (one
sample per bin, ``sampling_ratio`` ignored, box scaled by S/(S-1), zero padding, boxes divided by
``spatial_scale``).  Pinned by tests/golden/torch_function_c1.npz, which the reference module
itself produced (tests/golden/make_torch_function_golden.py).
"""
import torch
import torch.nn.functional as F


def roi_align_torch_function(feat_map, rois, output_size, spatial_scale=1.0, order=1, chunk=16):
    """feat_map (N, C, [D,] H, W); rois (R, 1 + 2*dim) = [batch, x1, y1, (z1,) x2, y2, (z2)].
    Returns (R, C, *output_size), float32 (roi_align.py:38-39 casts both inputs)."""
    feat_map = feat_map.float()
    rois = rois.float()
    mode = {1: 'bilinear', 0: 'nearest'}[order]
    dim = len(output_size)
    out = []
    for roi in rois:                                                      # roi_align.py:61-68
        batch_idx, box = int(roi[0]), roi[1:]
        feat = feat_map[batch_idx].unsqueeze(0)
        feat_size = torch.tensor(feat.shape[2:][::-1], dtype=torch.float32)
        x1 = box[:dim].unsqueeze(0) / spatial_scale                       # :93-94
        x2 = box[dim:].unsqueeze(0) / spatial_scale
        scaling = torch.diag_embed((x2 - x1) / (feat_size - 1))           # :100-101 (align_corners False)
        translation = ((x2 + x1 + 1) / feat_size - 1).unsqueeze(2)
        theta = torch.cat([scaling, translation], dim=-1)
        grids = torch.affine_grid_generator(theta, size=[1, feat.shape[1], *output_size], align_corners=False)
        out.append(torch.cat([F.grid_sample(feat, g, mode=mode, align_corners=False)
                              for g in torch.split(grids, chunk)]))
    return torch.cat(out, dim=0)


def config1_inputs(n_rois=128, seed=1):
    """RoIAlign 3D head configuration: features (2,4,64,64,64) uniform[0,1); rois with batch idx in {0,1}, centres
    uniform in the volume, side lengths uniform 8-48; output 7x7x7."""
    g = torch.Generator().manual_seed(seed)
    feat = torch.rand(2, 4, 64, 64, 64, generator=g)
    b = torch.randint(0, 2, (n_rois, 1), generator=g).float()
    c = torch.rand(n_rois, 3, generator=g) * 64
    s = torch.rand(n_rois, 3, generator=g) * 40 + 8
    return feat, torch.cat([b, c - s / 2, c + s / 2], 1)
