"""Seeded synthetic inputs of the five benchmark configurations (shapes, sizes and value
distributions of the reference's demos; the LUNA16 crops those use are not redistributable, so
CT-like random volumes stand in).  Shared by bench.py (what is timed) and tests/test_gpu_configs.py
(what is compared with the reference's own kernels), so that both run on the very same tensors.

Every generator returns a dict: name, features, rois (float32, on the CPU), out_size, and the
call's parameters (kind, sampling_ratio, aligned, order).
"""
import math

import torch

KIND_BOX, KIND_ROTATED = 0, 1
PATCH = 96


def ct_like(shape, seed, device):
    """int16 CT-like values ~N(-300,400) clipped to [-1024,3071], scaled to [0,1], fp16."""
    g = torch.Generator(device=device).manual_seed(seed)
    v = torch.empty(shape, device=device, dtype=torch.float32).normal_(-300, 400, generator=g)
    v = v.round_().clamp_(-1024, 3071)
    return ((v + 1024) / 4095).half()


def crop_rois(n_vol, per_vol, vol_shape, seed):
    """rois of CropRandomWithAffine (medvision/aug_cuda_batch/aug_spatial.py:674-715): random
    patch position, rotation about z within +-20 degrees, scale 0.9-1.1, no shift."""
    g = torch.Generator().manual_seed(seed)
    R = n_vol * per_vol
    D, H, W = vol_shape
    b = torch.arange(n_vol).repeat_interleave(per_vol).float().view(-1, 1)
    scale = torch.rand(R, 1, generator=g) * 0.2 + 0.9
    ext = torch.tensor([W, H, D], dtype=torch.float32)
    start = torch.rand(R, 3, generator=g) * (ext - PATCH)
    centre = start + PATCH / 2
    ang = torch.zeros(R, 3)
    ang[:, 2] = (torch.rand(R, generator=g) * 2 - 1) * math.radians(20)
    return torch.cat([b, centre, (PATCH / scale).expand(R, 3), ang], 1)


def workload_c1(device="cpu", rank=0, small=False, n_rois=128):
    """RoIAlign 3D head: features (2,4,64,64,64) fp32 uniform[0,1); rois with batch idx in {0,1},
    centres uniform in the volume, side lengths uniform 8-48; output 7x7x7, sampling_ratio 2."""
    g = torch.Generator().manual_seed(1 + rank)
    feat = torch.rand(2, 4, 64, 64, 64, generator=g)
    b = torch.randint(0, 2, (n_rois, 1), generator=g).float()
    c = torch.rand(n_rois, 3, generator=g) * 64
    s = torch.rand(n_rois, 3, generator=g) * 40 + 8
    return dict(name="RoIAlign 3D fp32 (2,4,64,64,64), %d rois, 7x7x7, sampling_ratio 2" % n_rois,
                features=feat.to(device), rois=torch.cat([b, c - s / 2, c + s / 2], 1), out_size=(7, 7, 7),
                kind=KIND_BOX, sampling_ratio=2, aligned=True, order=1)


def workload_c2(device="cpu", rank=0, small=False, dtype=torch.float32, n_rois=512):
    """RoIAlignRotated 2D head: features (8,3,512,512) ~N(0,1); rotated rois with centres uniform in
    the image, w/h uniform 16-256 px, angle uniform [-pi,pi); output 14x14, sampling_ratio 2."""
    g = torch.Generator().manual_seed(2 + rank)
    feat = torch.randn(8, 3, 512, 512, generator=g).to(dtype)
    b = torch.randint(0, 8, (n_rois, 1), generator=g).float()
    rois = torch.cat([b, torch.rand(n_rois, 2, generator=g) * 512, torch.rand(n_rois, 2, generator=g) * 240 + 16,
                      (torch.rand(n_rois, 1, generator=g) * 2 - 1) * math.pi], 1)
    return dict(name="RoIAlignRotated 2D %s (8,3,512,512), %d rois, 14x14, sampling_ratio 2" % (str(dtype)[6:], n_rois),
                features=feat.to(device), rois=rois, out_size=(14, 14), kind=KIND_ROTATED, sampling_ratio=2,
                aligned=True, order=1)


def workload_c3(device, rank=0, small=False):
    n = 1 if small else 4
    vol = ct_like((n, 1, 160, 512, 512), 3 + rank, device)
    rois = torch.tensor([[i, 256, 256, 80, 512, 512, 160, 0, 0, 0] for i in range(n)], dtype=torch.float32)
    return dict(name="Resize %dx(1,160,512,512) fp16 -> (128,256,256)" % n, features=vol, rois=rois,
                out_size=(128, 256, 256), kind=KIND_ROTATED, sampling_ratio=1, aligned=True, order=1)


def workload_c4(device, rank=0, small=False):
    n = 4 if small else 16
    g = torch.Generator(device=device).manual_seed(4 + rank)
    x = torch.empty((n, 1, 128, 128, 128), device=device).normal_(generator=g)
    k = torch.arange(-12, 13, device=device).float()
    k = torch.exp(-k * k / 32)
    k /= k.sum()
    for d in (2, 3, 4):  # separable Gaussian blur, sigma 4
        shp = [1, 1, 1, 1, 1]
        shp[d] = 25
        pad = [0, 0, 0]
        pad[d - 2] = 12
        x = torch.nn.functional.conv3d(x, k.view(shp), padding=pad)
    x = (x / x.std()).half()
    gc = torch.Generator().manual_seed(4 + rank)
    ang = (torch.rand(n, 3, generator=gc) * 2 - 1) * math.radians(30)
    sc = torch.rand(n, 1, generator=gc) * 0.4 + 0.8
    sh = (torch.rand(n, 3, generator=gc) * 2 - 1) * 10
    rois = torch.cat([torch.arange(n).float().view(-1, 1), 64 - sh / sc, (128 / sc).expand(n, 3), ang], 1)
    return dict(name="RandomAffine (%d,1,128,128,128) fp16, rotation +-30deg x3, scale 0.8-1.2, shift +-10" % n,
                features=x, rois=rois, out_size=(128, 128, 128), kind=KIND_ROTATED, sampling_ratio=1, aligned=True,
                order=1)


def workload_c5(device, rank=0, small=False):
    n_vol, per_vol = (2, 64) if small else (8, 64)
    shape = (1, 256, 512, 512)
    vol = ct_like((n_vol,) + shape, 5 + rank, device)
    rois = crop_rois(n_vol, per_vol, shape[1:], 5 + rank)
    return dict(name="CropRandomWithAffine %dx(1,256,512,512) fp16 -> (%d,1,96,96,96), z-rotation +-20deg, "
                     "scale 0.9-1.1" % (n_vol, n_vol * per_vol),
                features=vol, rois=rois, out_size=(PATCH,) * 3, kind=KIND_ROTATED, sampling_ratio=1, aligned=True,
                order=1)


WORKLOADS = {"c5": workload_c5, "c3": workload_c3, "c4": workload_c4}

# Distinct input elements read by the forward of the seeded workloads above, as counted on a B200 by the
# library's mark kernel: (workload, rank, small) -> U.  The benchmark's reference arm, which must not load the
# library, takes its algorithmic byte count from here; the library's own arm counts live and reports whether
# the two agree.
KNOWN_DISTINCT_INPUT_ELEMENTS = {
    ("c5", 0, False): 261262718,
    ("c5", 0, True): 67032018,
    ("c3", 0, False): 167772160,
    ("c4", 0, False): 25704429,
}
