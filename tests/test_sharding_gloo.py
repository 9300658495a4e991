"""The N > 1 path on CPU: two gloo ranks shard a job by sample, each computes its share with the
CPU restatement, and the gathered result equals the single-process result bit for bit -- the
path needs no data exchange."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from medvision_b200.sharding import max_over_ranks, partition, shard_by_sample


def test_partition_is_balanced_and_covers_everything():
    for n in (0, 1, 7, 8, 16, 513):
        for w in (1, 2, 3, 8):
            spans = [partition(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _job():
    g = torch.Generator().manual_seed(21)
    feat = torch.rand(5, 2, 6, 10, 12, generator=g).half()
    R = 11
    b = torch.randint(0, 5, (R, 1), generator=g).float()
    c = torch.rand(R, 3, generator=g) * torch.tensor([12., 10., 6.])
    s = torch.rand(R, 3, generator=g) * 6 + 2
    ang = torch.zeros(R, 3)
    ang[:, 2] = torch.rand(R, generator=g) - 0.5
    return feat, torch.cat([b, c, s, ang], 1).half()


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import port as oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    feat, rois = _job()
    f, r, pos = shard_by_sample(feat, rois, world, rank)
    out = oracle.forward(f, r, (3, 4, 5), oracle.KIND_ROTATED, 1.0, 1, True, 1, nthreads=1)
    gathered = [None] * world
    dist.all_gather_object(gathered, (pos, out))
    slowest = max_over_ranks(10.0 + rank)
    if rank == 0:
        full = torch.empty((rois.shape[0], 2, 3, 4, 5), dtype=torch.float16)
        for p, o in gathered:
            full[p] = o
        torch.save({"out": full, "slowest": slowest}, os.path.join(out_dir, "result.pt"))
    dist.destroy_process_group()


def test_two_ranks_equal_one(tmp_path):
    from oracle import port as oracle
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    res = torch.load(os.path.join(str(tmp_path), "result.pt"))
    feat, rois = _job()
    want = oracle.forward(feat, rois, (3, 4, 5), oracle.KIND_ROTATED, 1.0, 1, True, 1, nthreads=1)
    assert torch.equal(res["out"], want)
    assert res["slowest"] == 11.0


def test_shard_rebases_batch_index():
    feat, rois = _job()
    seen = 0
    for rank in range(3):
        f, r, pos = shard_by_sample(feat, rois, 3, rank)
        lo, hi = partition(5, 3, rank)
        assert f.shape[0] == hi - lo
        assert torch.all((r[:, 0] >= 0) & (r[:, 0] < hi - lo))
        assert torch.equal(r[:, 0].float() + lo, rois[pos, 0].float())
        seen += len(pos)
    assert seen == rois.shape[0]
