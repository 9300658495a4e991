"""Sharding of a resampling job over the GPUs of one node.

Every output element depends on ONE roi and on the (sample, channel) volume that roi names,
so the job splits by sample: a rank keeps a contiguous range of samples and exactly the rois
that point into it (their batch index rebased).  Nothing is exchanged on the data path; the
only communication a multi-GPU run needs is the gathering of results or timings on the host side
(``max_over_ranks``), which works over any torch.distributed backend.
"""
import torch


def partition(n_items, world_size, rank):
    """Contiguous, balanced range [lo, hi) of ``n_items`` for ``rank`` (the first ranks get the
    extra items)."""
    assert 0 <= rank < world_size
    base, extra = divmod(n_items, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_by_sample(features, rois, world_size, rank):
    """Local share of a job.

    Returns ``(features[lo:hi], local_rois, roi_positions)``: the samples of this rank, the rois
    whose batch index falls into [lo, hi) with that index rebased to the local batch, and their
    positions in the global roi list (so that results can be put back in order).
    """
    lo, hi = partition(features.shape[0], world_size, rank)
    b = rois[:, 0].to(torch.int64)
    keep = torch.nonzero((b >= lo) & (b < hi)).flatten()
    local = rois[keep].clone()
    local[:, 0] -= lo
    return features[lo:hi], local, keep


def max_over_ranks(value, device=None):
    """Largest ``value`` over the ranks of the default process group (itself without one)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
