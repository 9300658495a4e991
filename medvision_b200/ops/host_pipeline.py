"""Resampling of HOST-resident volumes, pipelined over the samples of the batch.

The reference's callers keep whole batches on the device (`image.cuda()` ... `affine_3d` ...
`.cpu()`), which serialises upload, kernel and download.  Every roi reads one sample only, so the
job splits by sample: while sample i is being resampled, sample i+1 is uploaded and the patches of
sample i-1 are downloaded -- three streams, two device buffers per direction.  PCIe carries both
directions at once, so the end-to-end time approaches max(upload, download) instead of their sum.

Results are identical to one `affine_3d` call on the whole batch (same kernel, same rois; only
the batch index is rebased per sample).  Streams, events and device buffers are kept per device
and shape and reused by later calls.
"""
import torch

from .. import _C

_SLOTS = 2


class _Pipe:
    """Streams, events and device buffers of one (device, sample shape, dtype, output shape) combination."""

    def __init__(self, device, sample_shape, dtype, max_r, channels, out_size):
        self.device = device
        self.max_r = max_r
        with torch.cuda.device(device):
            self.s_up, self.s_run, self.s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
            self.vol = [torch.empty((1,) + sample_shape, dtype=dtype, device=device) for _ in range(_SLOTS)]
            self.out = [torch.empty((max_r, channels) + out_size, dtype=dtype, device=device) for _ in range(_SLOTS)]
            self.up_done = [torch.cuda.Event() for _ in range(_SLOTS)]
            self.run_done = [torch.cuda.Event() for _ in range(_SLOTS)]
            self.down_done = [torch.cuda.Event() for _ in range(_SLOTS)]
            self.rois_dev = None
            self.rois_pin = None


_pipes = {}


def _pipe(device, sample_shape, dtype, max_r, channels, out_size):
    key = (device, sample_shape, dtype, channels, out_size)
    p = _pipes.get(key)
    if p is None or p.max_r < max_r:
        p = _pipes[key] = _Pipe(device, sample_shape, dtype, max_r, channels, out_size)
    return p


def affine_from_host(features, rois, out_size, spatial_scale=1.0, sampling_ratio=1, aligned=True, order=1,
                     device=None, out=None):
    """features: CPU tensor (N, C, [D,] H, W), ideally pinned; rois: CPU tensor (R, 6|10) with batch
    indices into ``features``; returns a pinned CPU tensor (R, C, *out_size) (``out`` if given).
    A roi whose batch index lies outside [0, N) yields zeros, as with the device-side call.
    Synchronises before returning."""
    assert not features.is_cuda and not rois.is_cuda, "host tensors expected"
    ndim = features.dim() - 2
    fn = _C.affine_2d if ndim == 2 else _C.affine_3d
    assert features.dtype in [torch.float32, torch.float16], f'input must be float16 or float32 but got {features.dtype}'
    assert order in [0, 1, 3], f'order {order} is not supported!'
    if order == 0:
        sampling_ratio = 1
    out_size = (out_size,) * ndim if isinstance(out_size, int) else tuple(int(v) for v in out_size)
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    N, C = features.shape[:2]
    R = rois.shape[0]
    if out is None:
        out = torch.empty((R, C) + out_size, dtype=features.dtype, pin_memory=True)
    if R == 0:
        return out
    batch = rois[:, 0].to(torch.int64)  # truncation towards zero, as the kernels read the index
    valid = (batch >= 0) & (batch < N)
    all_valid = bool(valid.all())
    if not all_valid:
        out[~valid] = 0
        batch = torch.where(valid, batch, torch.full_like(batch, N))  # sorted to the end, never launched
    order_idx = torch.argsort(batch, stable=True)
    counts = torch.bincount(batch, minlength=N + 1)[:N].tolist()
    contiguous = all_valid and bool(torch.equal(order_idx, torch.arange(R)))
    max_r = max(counts) if counts else 0
    if max_r == 0:
        return out
    pipe = _pipe(device, tuple(features.shape[1:]), features.dtype, max_r, C, out_size)
    with torch.cuda.device(device):
        cur = torch.cuda.current_stream()
        # rois: sorted by sample, batch index rebased to 0 (every launch sees a batch of one sample)
        n_valid = sum(counts)
        if pipe.rois_pin is None or pipe.rois_pin.shape[0] < R or pipe.rois_pin.shape[1] != rois.shape[1]:
            pipe.rois_pin = torch.empty((max(R, 64), rois.shape[1]), dtype=features.dtype, pin_memory=True)
            pipe.rois_dev = torch.empty_like(pipe.rois_pin, device=device)
        else:
            pipe.run_done[0].synchronize()  # the last kernels that read the roi buffer are done
            pipe.run_done[1].synchronize()
        pipe.rois_pin[:R].copy_(rois[order_idx])
        pipe.rois_pin[:R, 0] = 0
        for s in (pipe.s_up, pipe.s_run, pipe.s_down):
            s.wait_stream(cur)
        with torch.cuda.stream(pipe.s_up):
            pipe.rois_dev[:R].copy_(pipe.rois_pin[:R], non_blocking=True)
            rois_up = torch.cuda.Event()
            rois_up.record(pipe.s_up)
        pipe.s_run.wait_event(rois_up)
        stage = None if contiguous else torch.empty((n_valid, C) + out_size, dtype=features.dtype, pin_memory=True)
        target = out if contiguous else stage
        lo = 0
        for i in range(N):
            n_i = counts[i]
            if n_i == 0:
                continue
            k = i % _SLOTS
            with torch.cuda.stream(pipe.s_up):
                pipe.s_up.wait_event(pipe.run_done[k])      # the kernel that last read this slot is finished
                pipe.vol[k].copy_(features[i:i + 1], non_blocking=True)
                pipe.up_done[k].record(pipe.s_up)
            with torch.cuda.stream(pipe.s_run):
                pipe.s_run.wait_event(pipe.up_done[k])
                pipe.s_run.wait_event(pipe.down_done[k])    # the download that last read this out slot is finished
                fn(pipe.vol[k], pipe.rois_dev[lo:lo + n_i], pipe.out[k][:n_i], *out_size, spatial_scale, sampling_ratio,
                   aligned, order)
                pipe.run_done[k].record(pipe.s_run)
            with torch.cuda.stream(pipe.s_down):
                pipe.s_down.wait_event(pipe.run_done[k])
                target[lo:lo + n_i].copy_(pipe.out[k][:n_i], non_blocking=True)
                pipe.down_done[k].record(pipe.s_down)
            lo += n_i
        cur.wait_stream(pipe.s_down)
        cur.wait_stream(pipe.s_run)
        cur.wait_stream(pipe.s_up)
        torch.cuda.synchronize(device)
    if not contiguous:
        out[order_idx[:n_valid]] = stage
    return out
