"""Scene-parallel plumbing on CPU ranks (gloo, world size 2): sharding, the
batch-global serialization depth and the variable-length feature gather."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from pointtransformerv3_b200 import distributed as D
    try:
        counts = [5, 7, 3]
        off = torch.cumsum(torch.tensor(counts), 0)
        n = int(off[-1])
        data = dict(feat=torch.arange(n * 2, dtype=torch.float32).reshape(n, 2),
                    grid_coord=torch.arange(n * 3, dtype=torch.int32).reshape(n, 3) * (rank + 1),
                    coord=torch.zeros(n, 3), offset=off)
        lo, hi = D.shard_scenes(len(counts), rank, world)
        mine = D.slice_batch(data, lo, hi)
        assert mine["offset"].tolist() == torch.cumsum(torch.tensor(counts[lo:hi]), 0).tolist()
        assert mine["feat"].shape[0] == sum(counts[lo:hi])
        depth = D.global_depth(mine["grid_coord"])
        feats, rows = D.gather_features(mine["feat"] + 100 * rank)
        # the same with the counts supplied by the caller (no exchange of sizes)
        feats2, rows2 = D.gather_features(mine["feat"] + 100 * rank, counts=[12, 3])
        assert rows2 == rows and torch.equal(feats, feats2)
        try:
            D.gather_features(mine["feat"], counts=[1, 1])
            raise AssertionError("wrong counts must be refused")
        except ValueError:
            pass
        out.put((rank, lo, hi, depth, rows, feats.clone()))
    finally:
        dist.destroy_process_group()


def test_shard_depth_and_gather_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, lo0, hi0, d0, rows0, f0), (r1, lo1, hi1, d1, rows1, f1) = res
    assert (lo0, hi0, lo1, hi1) == (0, 2, 2, 3)            # contiguous scene groups covering the batch
    assert d0 == d1 == (44 * 2).bit_length()                # rank 1 holds the largest coordinate (44 * 2)
    assert rows0 == rows1 == [12, 3]
    assert torch.equal(f0, f1) and f0.shape == (15, 2)
    exp = torch.arange(30, dtype=torch.float32).reshape(15, 2)
    exp[12:] += 100
    assert torch.equal(f0, exp)


def test_shard_scenes_covers_everything():
    from pointtransformerv3_b200 import distributed as D
    for n in (1, 4, 16, 17):
        for world in (1, 2, 3, 8):
            spans = [D.shard_scenes(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


def test_shard_scenes_balanced():
    """Every scene goes to exactly one rank, every rank's list is ascending, and on sizes like those
    of the LiDAR batch the largest shard is closer to the mean than with equal scene counts."""
    from pointtransformerv3_b200 import distributed as D
    sizes = [135316, 135530, 121486, 107811, 133931, 141315, 134666, 147122, 143987, 135299, 117175, 144371,
             136325, 111214, 130525, 114574]
    for world in (1, 2, 4, 8, 16):
        groups = D.shard_scenes_balanced(sizes, world)
        assert len(groups) == world
        assert sorted(i for g in groups for i in g) == list(range(len(sizes)))
        assert all(g == sorted(g) for g in groups)
        assert groups == D.shard_scenes_balanced(sizes, world)            # the same on every rank
        load = [sum(sizes[i] for i in g) for g in groups]
        equal = [sum(sizes[slice(*D.shard_scenes(len(sizes), r, world))]) for r in range(world)]
        assert max(load) <= max(equal)
    groups = D.shard_scenes_balanced(sizes, 8)
    assert max(sum(sizes[i] for i in g) for g in groups) * 8 / sum(sizes) < 1.04
    # more ranks than scenes: the extra ranks get nothing
    assert sorted(map(len, D.shard_scenes_balanced([5, 3], 4))) == [0, 0, 1, 1]
