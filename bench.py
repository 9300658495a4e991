#!/usr/bin/env python
"""Benchmark of the resampling path: output Gvoxel/s of one forward pass of the batched
CropRandomWithAffine patch extraction (per GPU: 8 CT-like volumes (1,256,512,512) fp16,
64 rotated 96^3 patches per volume -> (512,1,96,96,96)), sharded over N GPUs by volume with
no communication, plus the roofline fraction of its kernel, CPU baselines and, at N = 1, the
Resize and RandomAffine configurations as extra lines of the same JSON object.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass of the path over the whole workload (one kernel launch per GPU).
Inputs are synthetic (seeded), already resident in HBM for `value`; `e2e` times the public
call with pinned HOST inputs and a host copy of the result inside the timed region.
Inputs (1.07 GB per GPU) are far larger than L2, so no explicit L2 flush is needed.

`--impl reference` runs the reference's own CUDA kernels (oracle/_ref, compiled unmodified for
sm_100a) on the same workload; if that build is absent it times the CPU restatement instead.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PATCH = 96


# ----------------------------------------------------------------------------- synthetic data
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


def workload_c5(device, rank, small=False):
    n_vol, per_vol = (2, 64) if small else (8, 64)
    shape = (1, 256, 512, 512)
    vol = ct_like((n_vol,) + shape, 5 + rank, device)
    rois = crop_rois(n_vol, per_vol, shape[1:], 5 + rank)
    return dict(name="CropRandomWithAffine %dx(1,256,512,512) fp16 -> (%d,1,96,96,96), z-rotation +-20deg, "
                     "scale 0.9-1.1" % (n_vol, n_vol * per_vol),
                features=vol, rois=rois, out_size=(PATCH,) * 3, order=1)


def workload_c3(device, rank, small=False):
    n = 1 if small else 4
    vol = ct_like((n, 1, 160, 512, 512), 3 + rank, device)
    rois = torch.tensor([[i, 256, 256, 80, 512, 512, 160, 0, 0, 0] for i in range(n)], dtype=torch.float32)
    return dict(name="Resize %dx(1,160,512,512) fp16 -> (128,256,256)" % n, features=vol, rois=rois,
                out_size=(128, 256, 256), order=1)


def workload_c4(device, rank, small=False):
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
                features=x, rois=rois, out_size=(128, 128, 128), order=1)


WORKLOADS = {"c5": workload_c5, "c3": workload_c3, "c4": workload_c4}

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per output voxel of this library's
# forward kernel, from one ncu capture of a reduced copy of the workload (profiles/); traffic grows
# in proportion to the voxels processed, so a launch's traffic is this figure times its outputs.
DRAM_BYTES_PER_OUTPUT_VOXEL = {"c5": 4.175, "c3": 10.6}


# ----------------------------------------------------------------------------- implementations
class Ours:
    name = "ours"

    def __init__(self):
        from medvision_b200 import _C
        from medvision_b200.ops import affine_3d
        self._C = _C
        self.affine_3d = affine_3d

    def forward_into(self, feat, rois, out, order):
        self._C.affine_3d(feat, rois, out, *out.shape[2:], 1.0, 1, True, order)

    def backward_into(self, grad, rois, gin, order):
        self._C.roi_align_rotated_3d_backward(grad, rois, gin, *grad.shape[2:], 1.0, 1, True, order)

    def public_forward(self, feat, rois, out_size, order):
        return self.affine_3d(feat, rois, tuple(out_size), 1.0, 1, True, order)

    def apply_offset(self, img, field, order):
        from medvision_b200.ops import apply_offset_3d
        return apply_offset_3d(img, field, order)

    def label_forward(self, seg, rois, out_size):
        from medvision_b200.ops import affine_label_3d
        return affine_label_3d(seg, rois, tuple(out_size))

    def forward2d_into(self, feat, rois, out, order):
        self._C.affine_2d(feat, rois, out, *out.shape[2:], 1.0, 1, True, order)

    def host_forward(self, feat_h, rois_h, out_size, order, out_h):
        """host tensors in, host tensor out: the library's pipelined entry point"""
        from medvision_b200.ops import affine_from_host
        return affine_from_host(feat_h, rois_h, tuple(out_size), 1.0, 1, True, order, out=out_h)


class ReferenceCuda:
    """The reference's own kernels (oracle/_ref), called like medvision/ops/cuda_fun_tools.py:48-91."""
    name = "reference"

    def __init__(self):
        from oracle import ref
        self.m = ref.module()

    def forward_into(self, feat, rois, out, order):
        self.m.affine_3d(feat, rois, out, *out.shape[2:], 1.0, 1, True, order)

    def backward_into(self, grad, rois, gin, order):
        self.m.roi_align_rotated_3d_backward(grad, rois, gin, *grad.shape[2:], 1.0, 1, True, order)

    def public_forward(self, feat, rois, out_size, order):
        out = feat.new_zeros((rois.size(0), feat.size(1)) + tuple(out_size))
        self.m.affine_3d(feat, rois.type(feat.type()), out, *out_size, 1.0, 1, True, order)
        return out

    def apply_offset(self, img, field, order):
        from oracle import ref
        return ref.apply_offset(img, field, order)

    def label_forward(self, seg, rois, out_size):
        """apply_to_seg of the reference's transforms (medvision/aug_cuda_batch/aug_spatial.py:158-194)"""
        return self.public_forward(seg.float(), rois, out_size, 0).int()

    def forward2d_into(self, feat, rois, out, order):
        self.m.affine_2d(feat, rois, out, *out.shape[2:], 1.0, 1, True, order)


# ----------------------------------------------------------------------------- measurement
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def window(self, t0, t1):
        """keep only the samples that arrived inside [t0, t1] (the timed region)"""
        self.t0, self.t1 = t0, t1

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        t0, t1 = getattr(self, "t0", 0.0), getattr(self, "t1", float("inf"))
        inside = [ln for ts, ln in self.lines if t0 <= ts <= t1 + 0.05]
        if not inside:  # region shorter than one sampling period: take the nearest samples
            inside = [ln for ts, ln in self.lines][-3:]
        for ln in inside:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x, world):
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return x


def time_steps(fn, steps, warmup, world):
    """W untimed steps, then exactly K steps between barrier + synchronize, timed with CUDA
    events on the launching (current) stream; returns ms for the K steps, max over ranks."""
    for _ in range(warmup):
        fn()
    barrier(world)
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world)


def touched_elements(feat, rois, out_size, order):
    """Exact count of distinct input elements read by the forward (mark pass, untimed)."""
    from medvision_b200 import _lib
    mask = torch.zeros(feat.shape, dtype=torch.uint8, device=feat.device)
    N, C, D, H, W = feat.shape
    rc = _lib.lib.mvr_roi_resample_touched(rois.data_ptr(), mask.data_ptr(), _lib.MVR_F16 if feat.dtype == torch.float16
                                           else _lib.MVR_F32, 3, _lib.MVR_ROI_ROTATED, N, C, D, H, W, rois.size(0),
                                           rois.size(1), *out_size, 1.0, 1, 1, order,
                                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.strerror(rc)
    total = 0
    for i in range(N):  # per volume: keeps the reduction's temporaries small
        total += int(mask[i].sum(dtype=torch.int64).item())
    return total


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def cpu_baseline_port(wl, budget_s=15.0):
    """The CPU restatement of the reference kernels on all host cores, on a bounded sample of the
    same workload: the rois of the first volumes, as many as fit the time budget."""
    from oracle import port
    rois_all = wl["rois"]
    threads = port.max_threads()
    feat0 = wl["features"][:1].cpu()
    probe = rois_all[rois_all[:, 0] == 0][:4].to(feat0.dtype).cpu()
    t0 = time.perf_counter()
    port.forward(feat0, probe, wl["out_size"], port.KIND_ROTATED, 1.0, 1, True, wl["order"])
    per_roi = (time.perf_counter() - t0) / max(1, probe.size(0))
    per_vol = int((rois_all[:, 0] == 0).sum())
    n_vol = int(max(1, min(wl["features"].size(0), budget_s / max(per_roi * per_vol, 1e-6))))
    feat = wl["features"][:n_vol].cpu()
    rois = rois_all[rois_all[:, 0] < n_vol].to(feat.dtype).cpu()
    t0 = time.perf_counter()
    out = port.forward(feat, rois, wl["out_size"], port.KIND_ROTATED, 1.0, 1, True, wl["order"])
    dt = time.perf_counter() - t0
    return {"value": out.numel() / dt / 1e9, "unit": "Gvoxel/s", "cores": threads, "kind": "port",
            "sample": "%d of %d rois (volumes 0..%d), %.1f s" % (rois.size(0), rois_all.size(0), n_vol - 1, dt)}


def cpu_baseline_torch_function():
    """The reference's torch-function RoIAlign path on CPU (restated in oracle/torch_function_path.py)
    on the RoIAlign 3D head configuration: features (2,4,64,64,64) fp32, 128 rois, output 7^3, forward + backward."""
    from oracle.torch_function_path import config1_inputs, roi_align_torch_function
    feat, rois = config1_inputs()
    feat.requires_grad_(True)
    g = torch.Generator().manual_seed(2)
    t0 = time.perf_counter()
    out = roi_align_torch_function(feat, rois, (7, 7, 7), 1.0, 1)
    t1 = time.perf_counter()
    out.backward(torch.randn(out.shape, generator=g))
    t2 = time.perf_counter()
    return {"unit": "Gvoxel/s", "cores": torch.get_num_threads(), "kind": "port of medvision/ops/pytorch_ops/roi_align.py",
            "sample": "config 1, 128 rois, whole", "fwd": out.numel() / (t1 - t0) / 1e9,
            "fwd_bwd": out.numel() / (t2 - t0) / 1e9, "fwd_ms": (t1 - t0) * 1e3, "bwd_ms": (t2 - t1) * 1e3}


def detection_configs(impl_name):
    """Latency of the small detection-style configurations (RoIAlign 3D and RoIAlignRotated 2D heads): forward and
    forward + backward through the op modules, CUDA events over 200 calls each."""
    if impl_name != "ours":
        return None
    from medvision_b200.ops import RoIAlign, RoIAlignRotated
    from oracle.torch_function_path import config1_inputs
    res = []

    def run(name, module, feat, rois, n_out):
        feat = feat.cuda().requires_grad_(True)
        rois = rois.cuda().to(feat.dtype)
        out = module(feat, rois)
        grad = torch.randn_like(out)
        for bwd in (False, True):
            def step():
                o = module(feat, rois)
                if bwd:
                    feat.grad = None
                    o.backward(grad)
            ms = time_steps(step, 200, 20, 1) / 200
            res.append({"workload": name, "pass": "fwd+bwd" if bwd else "fwd", "us_per_call": ms * 1e3,
                        "gvoxel_per_s": n_out / (ms * 1e-3) / 1e9, "note": "latency-bound; includes autograd and Python"})

    def run_graph(name, fwd_name, bwd_name, feat, rois, out_size, extra):
        """The two extension calls alone, replayed from a CUDA graph: launch and Python overhead removed."""
        from medvision_b200 import _C
        feat = feat.cuda()
        rois = rois.cuda().to(feat.dtype)
        out = torch.empty((rois.size(0), feat.size(1)) + tuple(out_size), dtype=feat.dtype, device="cuda")
        grad = torch.randn_like(out)
        gin = torch.zeros_like(feat)
        calls = {"fwd": lambda: getattr(_C, fwd_name)(feat, rois, out, *out_size, 1.0, 2, *extra, 1),
                 "bwd": lambda: getattr(_C, bwd_name)(grad, rois, gin, *out_size, 1.0, 2, *extra, 1)}
        for key, call in calls.items():
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                call()  # first call outside the capture (lazy set-up)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(20):
                        call()
            torch.cuda.synchronize()
            ms = time_steps(graph.replay, 20, 5, 1) / (20 * 20)
            res.append({"workload": name, "pass": key + " kernel, CUDA-graph replay", "us_per_call": ms * 1e3,
                        "gvoxel_per_s": out.numel() / (ms * 1e-3) / 1e9})

    feat, rois = config1_inputs()
    run_graph("RoIAlign 3D fp32 (2,4,64,64,64), 128 rois, 7x7x7, sampling_ratio 2", "roi_align_3d_forward",
              "roi_align_3d_backward", feat, rois, (7, 7, 7), ())
    run("RoIAlign 3D fp32 (2,4,64,64,64), 128 rois, 7x7x7, sampling_ratio 2",
        RoIAlign((7, 7, 7), 1.0, 2), feat, rois, 128 * 4 * 343)
    g = torch.Generator().manual_seed(2)
    for dt in (torch.float32, torch.float16):
        f2 = torch.randn(8, 3, 512, 512, generator=g).to(dt)
        b = torch.randint(0, 8, (512, 1), generator=g).float()
        r2 = torch.cat([b, torch.rand(512, 2, generator=g) * 512, torch.rand(512, 2, generator=g) * 240 + 16,
                        (torch.rand(512, 1, generator=g) * 2 - 1) * math.pi], 1)
        run("RoIAlignRotated 2D %s (8,3,512,512), 512 rois, 14x14, sampling_ratio 2" % str(dt)[6:],
            RoIAlignRotated((14, 14), 1.0, 2), f2, r2, 512 * 3 * 196)
        run_graph("RoIAlignRotated 2D %s (8,3,512,512), 512 rois, 14x14, sampling_ratio 2" % str(dt)[6:],
                  "roi_align_rotated_2d_forward", "roi_align_rotated_2d_backward", f2, r2, (14, 14), (True,))
    return res


def elastic_config(impl, peak):
    """The elastic deformation's two resampling steps on 4 CT-like half volumes (1,128,256,256):
    blowing the 8^3 control grid up to the dense displacement field (affine_3d, Catmull-Rom) and
    warping the image with it (apply_offset_3d, linear), as BatchCudaRandomElasticDeformation does."""
    shape = (4, 1, 128, 256, 256)
    img = ct_like(shape, 77, "cuda")
    g = torch.Generator().manual_seed(78)
    reach = torch.tensor([0.8 * n / 7 / 2 for n in shape[2:]]).reshape(1, 3, 1, 1, 1)
    coarse = (torch.rand((4, 3, 8, 8, 8), generator=g) * 2 - 1) * reach / 2
    for axis in (2, 3, 4):
        for pos in (0, 1, -1, -2):
            coarse.select(axis, pos).zero_()
    coarse = coarse.cuda()
    rois = torch.tensor([[b, 4, 4, 4, 5, 5, 5, 0, 0, 0] for b in range(4)], dtype=torch.float32).cuda()
    field = impl.public_forward(coarse, rois, shape[2:], 3)
    n = img.numel()
    res = []
    ms = time_steps(lambda: impl.public_forward(coarse, rois, shape[2:], 3), 20, 5, 1) / 20
    res.append({"workload": "elastic: control grid (4,3,8,8,8) fp32 -> dense field (4,3,128,256,256), affine_3d order 3",
                "pass": "fwd", "ms_per_step": ms, "gvoxel_per_s": field.numel() / (ms * 1e-3) / 1e9,
                "algorithmic_bytes": 4 * field.numel(), "achieved_gbs": 4 * field.numel() / (ms * 1e-3) / 1e9,
                "frac_of_peak": 4 * field.numel() / (ms * 1e-3) / 1e9 / peak, "note": "input fits in L1; store-bound"})
    ms = time_steps(lambda: impl.apply_offset(img, field, 1), 20, 5, 1) / 20
    # ours: the float field is read once and rounded to half in the kernel (3 x 4 B), image 2 B read, 2 B written;
    # the reference casts the field in a pass of its own first (3 x 4 B read, 3 x 2 B written, 3 x 2 B read again)
    alg = n * (3 * 4 + 2 + 2)
    res.append({"workload": "elastic: apply_offset_3d fp16 (4,1,128,256,256), fp32 field, linear", "pass": "fwd",
                "ms_per_step": ms, "gvoxel_per_s": n / (ms * 1e-3) / 1e9, "algorithmic_bytes": alg,
                "achieved_gbs": alg / (ms * 1e-3) / 1e9, "frac_of_peak": alg / (ms * 1e-3) / 1e9 / peak,
                "note": "public call; bytes = float field + half image read once, half result written once"})
    return res


def label_config(impl, peak):
    """The segmentation twin of the crop workload on a quarter of its size: 2 int32 label volumes
    (1,256,512,512), 128 rotated 96^3 patches, nearest, int32 result."""
    wl = workload_c5("cuda", 0, small=True)
    g = torch.Generator(device="cuda").manual_seed(9)
    seg = torch.randint(0, 6, tuple(wl["features"].shape), generator=g, device="cuda", dtype=torch.int32)
    rois = wl["rois"].float().cuda()
    out = impl.label_forward(seg, rois, wl["out_size"])
    ms = time_steps(lambda: impl.label_forward(seg, rois, wl["out_size"]), 20, 5, 1) / 20
    n = out.numel()
    U = touched_elements(wl["features"], wl["rois"].to(wl["features"].dtype).cuda(), wl["out_size"], 1)
    alg = 4 * n + 4 * U  # int32 result written once; at most the linear path's footprint read once
    return [{"workload": "label crops: 2x(1,256,512,512) int32 -> (128,1,96,96,96) int32, nearest", "pass": "fwd",
             "ms_per_step": ms, "gvoxel_per_s": n / (ms * 1e-3) / 1e9, "algorithmic_bytes": alg,
             "achieved_gbs": alg / (ms * 1e-3) / 1e9, "frac_of_peak": alg / (ms * 1e-3) / 1e9 / peak,
             "note": "public call; the reference arm runs seg.float() -> affine_3d(order 0) -> .int()"}]


def dense2d_config(impl, peak):
    """2D RandomAffine on 16 half images (1,2048,2048): rotation +-20 degrees, scale 0.9-1.1, shift +-10 px."""
    B, H, W = 16, 2048, 2048
    img = ct_like((B, 1, 1, H, W), 21, "cuda").reshape(B, 1, H, W)
    g = torch.Generator().manual_seed(22)
    scale = 0.9 + 0.2 * torch.rand(B, 1, generator=g)
    rois = torch.cat([torch.arange(B).float()[:, None],
                      torch.tensor([[W / 2, H / 2]]).repeat(B, 1) + (torch.rand(B, 2, generator=g) - 0.5) * 20,
                      torch.tensor([[float(W), float(H)]]).repeat(B, 1) / scale,
                      (torch.rand(B, 1, generator=g) - 0.5) * 0.7], 1).half().cuda()
    out = torch.empty_like(img)
    ms = time_steps(lambda: impl.forward2d_into(img, rois, out, 1), 50, 5, 1) / 50
    n = out.numel()
    alg = 2 * 2 * n  # every pixel read about once, every output written once
    return [{"workload": "2D RandomAffine: 16x(1,2048,2048) fp16 -> same, linear", "pass": "fwd", "ms_per_step": ms,
             "gvoxel_per_s": n / (ms * 1e-3) / 1e9, "algorithmic_bytes": alg, "achieved_gbs": alg / (ms * 1e-3) / 1e9,
             "frac_of_peak": alg / (ms * 1e-3) / 1e9 / peak, "note": "input larger than L2; issue-bound"}]


def cpu_baseline_scipy():
    """What the reference's numpy augmentations call for the same job
    (medvision/aug_cpu/aug_spatial.py:475 rotate, :99 zoom), single-threaded scipy."""
    try:
        import numpy as np
        import scipy.ndimage as ndi
    except ImportError:
        return None
    rng = np.random.default_rng(0)
    v = rng.random((1, PATCH, PATCH, PATCH), dtype=np.float32)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 2.0:
        ndi.rotate(v, 15.0, axes=(3, 2), reshape=False, order=1, mode="constant", cval=0)
        reps += 1
    rot = reps * v.size / (time.perf_counter() - t0) / 1e9
    t0 = time.perf_counter()
    ndi.zoom(v, (1, 1.1, 1.1, 1.1), order=2)
    zoom = v.size * 1.1 ** 3 / (time.perf_counter() - t0) / 1e9
    return {"unit": "Gvoxel/s", "cores": 1, "kind": "scipy.ndimage calls of the reference's aug_cpu",
            "rotate_order1": rot, "zoom_order2": zoom, "sample": "(1,96,96,96) float32 patch"}


def measure(impl, wl, steps, warmup, world, backward=False):
    feat, rois = wl["features"], wl["rois"].to(wl["features"].dtype).cuda()
    out = torch.empty((rois.size(0), feat.size(1)) + tuple(wl["out_size"]), dtype=feat.dtype, device="cuda")
    if not backward:
        ms = time_steps(lambda: impl.forward_into(feat, rois, out, wl["order"]), steps, warmup, world)
        return ms / steps, out
    g = torch.Generator(device="cuda").manual_seed(1)
    grad = torch.empty_like(out).normal_(generator=g)
    gin = torch.empty_like(feat)

    def step():
        impl.forward_into(feat, rois, out, wl["order"])
        gin.zero_()  # part of every backward: the op accumulates into a zeroed gradient
        impl.backward_into(grad, rois, gin, wl["order"])
    ms = time_steps(step, steps, warmup, world)
    return ms / steps, out


def measure_e2e(impl, wl, steps, warmup, world):
    """Public call with HOST buffers: pinned inputs -> device, resample, result -> pinned host."""
    feat_h = wl["features"].cpu().pin_memory()
    rois_h = wl["rois"].pin_memory()
    out_shape = (rois_h.size(0), feat_h.size(1)) + tuple(wl["out_size"])
    out_h = torch.empty(out_shape, dtype=feat_h.dtype).pin_memory()

    def step():
        if hasattr(impl, "host_forward"):
            impl.host_forward(feat_h, rois_h, wl["out_size"], wl["order"], out_h)
            return
        f = feat_h.cuda(non_blocking=True)
        r = rois_h.cuda(non_blocking=True)
        o = impl.public_forward(f, r, wl["out_size"], wl["order"])
        out_h.copy_(o, non_blocking=True)
    ms = time_steps(step, steps, warmup, world) / steps
    h2d = feat_h.numel() * feat_h.element_size() + rois_h.numel() * rois_h.element_size()
    d2h = out_h.numel() * out_h.element_size()
    return ms, h2d, d2h, out_h


def run_cpu_reference(args, rank):
    """Fallback of --impl reference when the reference's CUDA build is absent: the CPU
    restatement with all host threads on a bounded sample per step."""
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]("cpu", 0, small=True)
    base = cpu_baseline_port(wl, budget_s=8.0)
    line = {"impl": "reference", "metric": "resampled Gvoxel/s (fwd)", "value": base["value"], "unit": "Gvoxel/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": wl["name"], "device": "cpu"}, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "Gvoxel/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["elastic", "det"], default="c5",
                    help="elastic / det: only the elastic, label and 2D entries / only the detection-head "
                         "configurations of other_configs, one GPU (profiling aids)")
    ap.add_argument("--small", action="store_true", help="reduced copy of the workload (for profiler captures)")
    ap.add_argument("--kernel-only", action="store_true", help="skip e2e, CPU baselines and the extra configurations")
    ap.add_argument("--backward", action="store_true", help="time forward + backward instead of forward (profiling aid)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        from oracle import ref
        if not (ref.available() and torch.cuda.is_available()):
            run_cpu_reference(args, int(os.environ.get("RANK", "0")))
            return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: medvision_b200 has no CPU path")

    rank, world, local = dist_setup(args.gpus)
    impl = Ours() if args.impl == "ours" else ReferenceCuda()
    if args.workload == "det":
        if rank == 0:
            print(json.dumps({"impl": args.impl, "detection": detection_configs(args.impl)}))
        return
    if args.workload == "elastic":
        if rank == 0:
            print(json.dumps({"impl": args.impl, "elastic": elastic_config(impl, load_peaks()[0]),
                              "label": label_config(impl, load_peaks()[0]),
                              "dense2d": dense2d_config(impl, load_peaks()[0])}))
        return
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # started early: the tool needs a moment before its first sample
    wl = WORKLOADS[args.workload]("cuda", rank, small=args.small)
    n_out = wl["rois"].size(0) * wl["features"].size(1) * math.prod(wl["out_size"])

    t_begin = time.time()
    ms, out = measure(impl, wl, args.steps, args.warmup, world, backward=args.backward)
    sampler.window(t_begin, time.time())
    clocks = sampler.stop() if rank == 0 else None
    value = world * n_out / (ms * 1e-3) / 1e9

    line = {"metric": "resampled Gvoxel/s (fwd)", "value": value, "unit": "Gvoxel/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": wl["name"], "sharding": "by volume, %d GPU(s), no collective" % world,
                       "l2": "inputs (%.2f GB per GPU) larger than L2, no flush" %
                             (wl["features"].numel() * 2 / 1e9),
                       "sampling_ratio": 1, "order": 1, "aligned": True},
            "gpu_launches": (2 if args.impl == "ours" else 1) * args.steps, "clocks": clocks}
    if args.impl == "reference":
        line["impl"] = "reference"
        line["config"]["device"] = "cuda: the reference's own kernels, compiled unmodified for sm_100a"

    # roofline of the dominant (only) kernel: algorithmic bytes / measured launch duration
    e = wl["features"].element_size()
    rois_dev = wl["rois"].to(wl["features"].dtype).cuda()
    U = touched_elements(wl["features"], rois_dev, wl["out_size"], wl["order"])
    alg_bytes = e * (U + n_out) + rois_dev.numel() * e
    peak, peak_src = load_peaks()
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "traffic": (DRAM_BYTES_PER_OUTPUT_VOXEL.get(args.workload) * n_out
                                    if args.impl == "ours" and DRAM_BYTES_PER_OUTPUT_VOXEL.get(args.workload) else None),
                        "peak_source": peak_src, "algorithmic_bytes_per_launch": alg_bytes,
                        "distinct_input_elements": U, "output_elements": n_out,
                        "frac_of_8000_nominal": achieved / 8000.0}

    if not args.kernel_only:
        ems, h2d, d2h, _ = measure_e2e(impl, wl, max(2, min(args.steps // 4, 10)), 3, world)
        line["e2e"] = {"value": world * n_out / (ems * 1e-3) / 1e9, "unit": "Gvoxel/s", "ms_per_step": ems,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        if args.impl == "reference" and rank == 0:
            line["cpu_baseline"] = {"value": value, "unit": "Gvoxel/s", "cores": 0, "kind": "reference",
                                    "sample": "whole workload on the GPU (the reference path has no CPU implementation)"}
        if world == 1 and args.impl == "ours":
            line["cpu_baseline"] = cpu_baseline_port(wl)
            sp = cpu_baseline_scipy()
            if sp:
                line["cpu_baseline_aug_cpu"] = sp
            line["cpu_baseline_torch_function"] = cpu_baseline_torch_function()
        if world == 1 and args.workload == "c5" and not args.small:
            extra = []
            del out
            wl = None
            torch.cuda.empty_cache()
            for key, bwd in (("c3", False), ("c4", False), ("c4", True)):
                w2 = WORKLOADS[key]("cuda", 0)
                n2 = w2["rois"].size(0) * math.prod(w2["out_size"])
                m2, _ = measure(impl, w2, min(max(args.steps, 20), 100), min(args.warmup, 10), 1, backward=bwd)
                r2 = w2["rois"].to(w2["features"].dtype).cuda()
                U2 = touched_elements(w2["features"], r2, w2["out_size"], 1)
                b2 = 2 * (U2 + n2) + r2.numel() * 2
                if bwd:
                    b2 += 2 * (n2 + w2["features"].numel()) + r2.numel() * 2
                extra.append({"workload": w2["name"], "pass": "fwd+bwd" if bwd else "fwd", "ms_per_step": m2,
                              "gvoxel_per_s": n2 / (m2 * 1e-3) / 1e9, "algorithmic_bytes": b2,
                              "achieved_gbs": b2 / (m2 * 1e-3) / 1e9, "frac_of_peak": b2 / (m2 * 1e-3) / 1e9 / peak,
                              "note": "input fits in L2" if key == "c4" else "input larger than L2"})
            extra += elastic_config(impl, peak)
            extra += label_config(impl, peak)
            extra += dense2d_config(impl, peak)
            det = detection_configs(args.impl)
            if det:
                extra += det
            line["other_configs"] = extra
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
