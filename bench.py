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

from bench_workloads import (KNOWN_DISTINCT_INPUT_ELEMENTS, PATCH, WORKLOADS, ct_like, workload_c1,  # noqa: E402
                             workload_c2, workload_c5)

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per output voxel of this library's
# forward kernel, from one ncu capture of a reduced copy of the workload (profiles/); traffic grows
# in proportion to the voxels processed, so a launch's traffic is this figure times its outputs.
DRAM_BYTES_PER_OUTPUT_VOXEL = {
    "c5": {"bytes": 4.175, "source": "profiles/fwd_stream3d_tma_half_c5_small.md (ncu, 2-volume copy of the workload)"},
    "c3": {"bytes": 10.6, "source": "profiles/fwd_stream3d_tma_half_c3_small.md (ncu, 1-volume copy of the workload)"},
}


# ----------------------------------------------------------------------------- implementations
class Ours:
    name = "ours"

    def __init__(self):
        from medvision_b200 import _C
        from medvision_b200.ops import affine_3d
        self._C = _C
        self.affine_3d = affine_3d

    def raw(self, name):
        """the extension function `name` (same names and arguments in both arms)"""
        return getattr(self._C, name)

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

    def raw(self, name):
        return getattr(self.m, name)

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


def distinct_inputs(impl, key, rank, small, feat, rois, out_size, order=1):
    """U of a workload: counted live by this library's mark kernel in its own arm; the reference arm must load
    nothing of this library and takes the committed count of the same seeded tensors (None if there is none)."""
    known = KNOWN_DISTINCT_INPUT_ELEMENTS.get((key, rank, bool(small)))
    if impl.name != "ours":
        return known, known
    return touched_elements(feat, rois, out_size, order), known


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
    from oracle.torch_function_path import roi_align_torch_function
    w1 = workload_c1()
    feat, rois = w1["features"], w1["rois"]
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


def detection_configs(impl):
    """Latency of the small detection-style configurations (RoIAlign 3D and RoIAlignRotated 2D heads).  Both arms:
    the two extension calls alone, 200 back-to-back launches between CUDA events (the kernels outlast their launch
    cost, so this is kernel time).  This library also: the same calls replayed from a CUDA graph (the reference
    launches on the legacy default stream, which cannot be captured), and forward / forward + backward through the
    op modules with autograd and Python included."""
    res = []
    ours = impl.name == "ours"

    def run_modules(name, module, feat, rois, n_out):
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

    def run_kernels(w, fwd_name, bwd_name, extra):
        feat = w["features"].cuda()
        rois = w["rois"].cuda().to(feat.dtype)
        out_size = tuple(w["out_size"])
        out = torch.empty((rois.size(0), feat.size(1)) + out_size, dtype=feat.dtype, device="cuda")
        grad = torch.randn_like(out)
        gin = torch.zeros_like(feat)
        fwd, bwd = impl.raw(fwd_name), impl.raw(bwd_name)
        calls = {"fwd": lambda: fwd(feat, rois, out, *out_size, 1.0, w["sampling_ratio"], *extra, 1),
                 "bwd": lambda: bwd(grad, rois, gin, *out_size, 1.0, w["sampling_ratio"], *extra, 1)}
        for key, call in calls.items():
            ms = time_steps(call, 200, 20, 1) / 200
            res.append({"workload": w["name"], "pass": key + " kernel, back-to-back launches", "us_per_call": ms * 1e3,
                        "gvoxel_per_s": out.numel() / (ms * 1e-3) / 1e9})
            if not ours:
                continue
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
            res.append({"workload": w["name"], "pass": key + " kernel, CUDA-graph replay", "us_per_call": ms * 1e3,
                        "gvoxel_per_s": out.numel() / (ms * 1e-3) / 1e9})

    w1 = workload_c1()
    run_kernels(w1, "roi_align_3d_forward", "roi_align_3d_backward", ())
    if ours:
        from medvision_b200.ops import RoIAlign, RoIAlignRotated
        run_modules(w1["name"], RoIAlign((7, 7, 7), 1.0, 2), w1["features"], w1["rois"], 128 * 4 * 343)
    for dt in (torch.float32, torch.float16):
        w2 = workload_c2(dtype=dt)
        run_kernels(w2, "roi_align_rotated_2d_forward", "roi_align_rotated_2d_backward", (True,))
        if ours:
            run_modules(w2["name"], RoIAlignRotated((14, 14), 1.0, 2), w2["features"], w2["rois"], 512 * 3 * 196)
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
    U, _ = distinct_inputs(impl, "c5", 0, True, wl["features"], wl["rois"].to(wl["features"].dtype).cuda(), wl["out_size"])
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

    # The box's copy ceiling for this step: the same bytes, pinned host <-> device, both directions at
    # once on two streams, no kernel, every rank at the same time (they share the host's memory and
    # PCIe paths).  e2e cannot be faster than this; e2e / ceiling says how much of it is overhead.
    dev_in = torch.empty_like(feat_h, device="cuda")
    dev_out = torch.empty(out_shape, dtype=feat_h.dtype, device="cuda")
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def copies_only():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            dev_in.copy_(feat_h, non_blocking=True)
        with torch.cuda.stream(s_out):
            out_h.copy_(dev_out, non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
    ceil_ms = time_steps(copies_only, steps, 2, world) / steps
    return ms, h2d, d2h, ceil_ms


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
            "config": {"workload": wl["name"]}, "reference_runs_on": "cpu restatement (oracle/_ref absent)",
            "cpu_baseline": base,
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
            print(json.dumps({"impl": args.impl, "detection": detection_configs(impl)}))
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
        line["reference_runs_on"] = "cuda: the reference's own kernels, compiled unmodified for sm_100a"

    # roofline of the dominant (only) kernel: algorithmic bytes / measured launch duration.  U (distinct
    # input elements read) is counted by this library's mark kernel in its own arm; the reference arm
    # loads nothing of this library and takes the committed count of the same seeded workload.
    e = wl["features"].element_size()
    rois_dev = wl["rois"].to(wl["features"].dtype).cuda()
    U, known_u = distinct_inputs(impl, args.workload, rank, args.small, wl["features"], rois_dev, wl["out_size"],
                                 wl["order"])
    peak, peak_src = load_peaks()
    if U is not None:
        alg_bytes = e * (U + n_out) + rois_dev.numel() * e
        achieved = alg_bytes / (ms * 1e-3) / 1e9
        per_voxel = DRAM_BYTES_PER_OUTPUT_VOXEL.get(args.workload) if args.impl == "ours" else None
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                            "traffic": per_voxel["bytes"] * n_out if per_voxel else None,
                            "traffic_source": per_voxel["source"] if per_voxel else None,
                            "peak_source": peak_src, "algorithmic_bytes_per_launch": alg_bytes,
                            "distinct_input_elements": U, "output_elements": n_out,
                            "distinct_input_elements_match_committed": (U == known_u) if known_u else None,
                            "frac_of_8000_nominal": achieved / 8000.0}

    if not args.kernel_only:
        ems, h2d, d2h, ceil_ms = measure_e2e(impl, wl, max(2, min(args.steps // 4, 10)), 3, world)
        line["e2e"] = {"value": world * n_out / (ems * 1e-3) / 1e9, "unit": "Gvoxel/s", "ms_per_step": ems,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "h2d_gbs_per_rank": h2d / (ems * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (ems * 1e-3) / 1e9,
                       "copy_ceiling_ms": ceil_ms, "frac_of_copy_ceiling": ceil_ms / ems,
                       "copy_ceiling": "the same bytes per step and rank as plain pinned copies in both directions at "
                                       "once, no kernel, all %d rank(s) together; max over ranks" % world,
                       "copy_ceiling_h2d_gbs_per_rank": h2d / (ceil_ms * 1e-3) / 1e9,
                       "copy_ceiling_d2h_gbs_per_rank": d2h / (ceil_ms * 1e-3) / 1e9}
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
                U2, _ = distinct_inputs(impl, key, 0, False, w2["features"], r2, w2["out_size"])
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
            extra += detection_configs(impl)
            line["other_configs"] = extra
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
