"""Resampling of HOST-resident volumes, pipelined over the samples of the batch.

The reference's callers keep whole batches on the device (`image.cuda()` ... `affine_3d` ...
`.cpu()`), which serialises upload, kernel and download.  Every roi reads one sample only, so the
job splits by sample: while sample i is being resampled, sample i+1 is uploaded and the patches of
sample i-1 are downloaded -- three streams, two device buffers per direction.  PCIe carries both
directions at once, so the end-to-end time approaches max(upload, download) instead of their sum.

Results are identical to one `affine_3d` call on the whole batch (same kernel, same rois; only
the batch index is rebased per sample).
"""
import torch

from .. import _C


def affine_from_host(features, rois, out_size, spatial_scale=1.0, sampling_ratio=1, aligned=True, order=1,
                     device=None, out=None):
    """features: CPU tensor (N, C, [D,] H, W), ideally pinned; rois: CPU tensor (R, 6|10) with batch
    indices into ``features``; returns a pinned CPU tensor (R, C, *out_size) (``out`` if given).
    Synchronises before returning."""
    assert not features.is_cuda and not rois.is_cuda, "host tensors expected"
    ndim = features.dim() - 2
    fn = _C.affine_2d if ndim == 2 else _C.affine_3d
    assert features.dtype in [torch.float32, torch.float16], f'input must be float16 or float32 but got {features.dtype}'
    assert order in [0, 1], f'order {order} is not supported!'
    if order == 0:
        sampling_ratio = 1
    out_size = (out_size,) * ndim if isinstance(out_size, int) else tuple(out_size)
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    N, C = features.shape[:2]
    R = rois.shape[0]
    if out is None:
        out = torch.empty((R, C) + out_size, dtype=features.dtype, pin_memory=True)
    batch = rois[:, 0].to(torch.int64)
    order_idx = torch.argsort(batch, stable=True)
    counts = torch.bincount(batch, minlength=N).tolist()
    contiguous = bool(torch.equal(order_idx, torch.arange(R)))
    rois_sorted = rois[order_idx].to(features.dtype).clone()
    rois_sorted[:, 0] = 0  # every launch sees a batch of one sample
    max_r = max(counts) if counts else 0
    with torch.cuda.device(device):
        s_up, s_run, s_down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        cur = torch.cuda.current_stream()
        for s in (s_up, s_run, s_down):
            s.wait_stream(cur)
        rois_dev = rois_sorted.pin_memory().to(device, non_blocking=True) if R else rois_sorted.to(device)
        s_up.wait_stream(cur)
        slots = 2
        vol_buf = [torch.empty((1,) + tuple(features.shape[1:]), dtype=features.dtype, device=device)
                   for _ in range(slots)]
        out_buf = [torch.empty((max_r, C) + out_size, dtype=features.dtype, device=device) for _ in range(slots)]
        up_done = [torch.cuda.Event() for _ in range(slots)]
        run_done = [torch.cuda.Event() for _ in range(slots)]
        down_done = [torch.cuda.Event() for _ in range(slots)]
        stage = None if contiguous else torch.empty_like(out)  # results in sorted roi order
        target = out if contiguous else stage
        lo = 0
        for i in range(N):
            k = i % slots
            n_i = counts[i]
            if n_i == 0:
                continue
            with torch.cuda.stream(s_up):
                s_up.wait_event(run_done[k])      # the kernel that last read this slot is finished
                vol_buf[k].copy_(features[i:i + 1], non_blocking=True)
                up_done[k].record(s_up)
            with torch.cuda.stream(s_run):
                s_run.wait_event(up_done[k])
                s_run.wait_event(down_done[k])    # the download that last read this out slot is finished
                fn(vol_buf[k], rois_dev[lo:lo + n_i], out_buf[k][:n_i], *out_size, spatial_scale, sampling_ratio,
                   aligned, order)
                run_done[k].record(s_run)
            with torch.cuda.stream(s_down):
                s_down.wait_event(run_done[k])
                target[lo:lo + n_i].copy_(out_buf[k][:n_i], non_blocking=True)
                down_done[k].record(s_down)
            lo += n_i
        cur.wait_stream(s_down)
        cur.wait_stream(s_run)
        cur.wait_stream(s_up)
        torch.cuda.synchronize(device)
    if not contiguous:
        out[order_idx] = stage
    return out
