"""Bit-exact parity of the CUDA serialization stage (codes, stable sort order,
inverse) with the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import cenc
from oracle import ptv3_oracle as O
from pointtransformerv3_b200 import ops, synthetic

pytestmark = pytest.mark.gpu
ORDERS = ["z", "z-trans", "hilbert", "hilbert-trans"]


def _check_sorted(codes, order, inverse):
    k, n = codes.shape
    ar = torch.arange(n, device=codes.device)
    for r in range(k):
        sc = codes[r][order[r]]
        assert bool((sc[1:] >= sc[:-1]).all())
        tie = sc[1:] == sc[:-1]
        assert bool((order[r][1:][tie] > order[r][:-1][tie]).all()), "ties must keep index order"
        assert bool((inverse[r][order[r]] == ar).all())


@pytest.mark.parametrize("depth", [1, 2, 5, 8, 9, 11, 16])
def test_encode_matches_oracle(depth):
    rng = np.random.default_rng(depth)
    g = rng.integers(-3, (1 << depth) + 3, size=(5000, 3)).astype(np.int32)
    b = rng.integers(0, 5, size=5000).astype(np.int64)
    got = ops.encode(torch.from_numpy(g).cuda(), torch.from_numpy(b).cuda(), depth, ORDERS).cpu().numpy()
    for r, o in enumerate(ORDERS):
        assert (got[r] == cenc.encode(g, b, depth, o)).all(), o


def test_encode_edge_sizes():
    for n in (0, 1, 2, 31, 257):
        g = torch.randint(0, 1 << 16, (n, 3), dtype=torch.int32)
        got = ops.encode(g.cuda(), None, 16, ORDERS).cpu().numpy()
        assert got.shape == (4, n)
        for r, o in enumerate(ORDERS):
            assert (got[r] == cenc.encode(g.numpy(), None, 16, o)).all()


def test_config1_bit_exact():
    """100 000 uniform points, depth 16, four orders: codes, order, inverse."""
    _, gc = synthetic.uniform_cloud(100_000, seed=0)
    batch = torch.zeros(gc.shape[0], dtype=torch.int64)
    codes = ops.encode(gc.cuda(), batch.cuda(), 16, ORDERS)
    order, inverse = ops.argsort_inverse(codes, 48 + 1)
    c = codes.cpu().numpy()
    for r, o in enumerate(ORDERS):
        ref = cenc.encode(gc.numpy(), batch.numpy(), 16, o)
        assert (c[r] == ref).all()
        ro = cenc.argsort_stable(ref)
        assert (order[r].cpu().numpy() == ro).all()
        assert (inverse[r].cpu().numpy() == cenc.inverse(ro)).all()


@pytest.mark.parametrize("n,bits", [(1, 8), (2, 3), (33, 1), (2048, 16), (2049, 17), (70_001, 30),
                                    (300_000, 38), (1_000_000, 63)])
def test_argsort_sizes_and_ties(n, bits):
    g = torch.Generator().manual_seed(n)
    hi = (1 << bits) - 1
    codes = torch.randint(0, min(hi, 1 << 62) + 1, (3, n), generator=g, dtype=torch.int64)
    codes[1] = codes[1] % 7          # heavy ties
    codes[2] = torch.sort(codes[2], descending=True).values
    order, inverse = ops.argsort_inverse(codes.cuda(), bits)
    _check_sorted(codes.cuda(), order, inverse)
    for r in range(3):
        assert (order[r].cpu().numpy() == np.argsort(codes[r].numpy(), kind="stable")).all()


def test_large_sort_properties():
    """4 M points x 4 orders: sortedness, stability and inverse, checked on device."""
    n = 4_000_000
    g = torch.Generator(device="cuda").manual_seed(0)
    gc = torch.randint(0, 2048, (n, 3), generator=g, device="cuda", dtype=torch.int32)
    batch = torch.randint(0, 16, (n,), generator=g, device="cuda").sort().values
    codes = ops.encode(gc, batch, 11, ORDERS)
    order, inverse = ops.argsort_inverse(codes, 33 + 4)
    _check_sorted(codes, order, inverse)


@pytest.mark.parametrize("depth", [1, 4, 9, 16])
def test_decode_inverts_encode(depth):
    """serialization.decode for "z" and "hilbert": coordinates and scene ids back."""
    from pointtransformerv3_b200 import serialization
    rng = np.random.default_rng(depth)
    g = rng.integers(0, 1 << depth, size=(4000, 3)).astype(np.int32)
    b = rng.integers(0, 6, size=4000).astype(np.int64)
    for name in ("z", "hilbert"):
        code = serialization.encode(torch.from_numpy(g).cuda(), torch.from_numpy(b).cuda(), depth, name)
        grid, batch = serialization.decode(code, depth, name)
        assert grid.dtype == torch.int64 and grid.shape == (4000, 3)
        assert (grid.cpu().numpy() == g).all() and (batch.cpu().numpy() == b).all()
        og, ob = cenc.decode(code.cpu().numpy(), depth, name)
        assert (grid.cpu().numpy() == og).all() and (batch.cpu().numpy() == ob).all()


@pytest.mark.gpu
@pytest.mark.parametrize("n,scenes", [(1, 1), (5000, 1), (40_000, 3), (300_000, 4)])
def test_grid_coord_and_voxel_dedup_match_oracle(n, scenes):
    """Bit-exact: grid coordinates (model.py:94-96) and first-point-per-voxel selection."""
    from pointtransformerv3_b200 import ops
    g = torch.Generator().manual_seed(n)
    coord = (torch.rand(n, 3, generator=g) * torch.tensor([8.0, 6.0, 3.0]) - torch.tensor([2.0, 0.5, 1.0]))
    if n > 100:
        coord[50:100] = coord[0:50]                      # exact duplicates
    cuts = sorted(torch.randint(0, n + 1, (scenes - 1,), generator=g).tolist()) + [n]
    offset = torch.tensor(cuts, dtype=torch.int64)       # ragged, possibly empty scenes
    grid_size = 0.04
    ref_grid = O.grid_coord_from_coord(coord, grid_size)
    grid, origin = ops.grid_coord(coord.cuda(), grid_size)
    assert torch.equal(grid.cpu(), ref_grid)
    assert torch.equal(origin.cpu(), coord.min(0)[0])
    batch = O.offset_to_batch(offset)
    ind = torch.cat([batch.unsqueeze(-1).int(), ref_grid], 1).contiguous()
    d = ops.voxel_dedup(ind.cuda(), offset.cuda())
    keep, p2v, off = O.voxel_dedup(batch, ref_grid, offset)
    assert d["m"] == keep.numel()
    assert torch.equal(d["keep"].cpu(), keep)
    assert torch.equal(d["point2voxel"].cpu(), p2v)
    assert torch.equal(d["offset"].cpu(), off)
    # idempotence: the kept points are already one per voxel
    d2 = ops.voxel_dedup(ind.cuda().index_select(0, d["keep"]), d["offset"])
    assert d2["m"] == d["m"] and torch.equal(d2["keep"].cpu(), torch.arange(d["m"]))


@pytest.mark.gpu
def test_voxelize_feeds_the_backbone():
    """Raw points -> voxelize -> backbone: same features as the backbone run on the
    oracle's selection of points."""
    import pointtransformerv3_b200 as P
    g = torch.Generator().manual_seed(3)
    n = 30_000
    coord = torch.rand(n, 3, generator=g) * torch.tensor([3.0, 3.0, 1.0])
    feat = torch.cat([coord, torch.rand(n, 3, generator=g)], 1)
    offset = torch.tensor([17_000, n])
    data, p2v = P.voxelize(coord.cuda(), feat.cuda(), offset.cuda(), 0.02)
    ref_grid = O.grid_coord_from_coord(coord, 0.02)
    keep, ref_p2v, ref_off = O.voxel_dedup(O.offset_to_batch(offset), ref_grid, offset)
    assert torch.equal(data["grid_coord"].cpu(), ref_grid[keep]) and torch.equal(data["offset"].cpu(), ref_off)
    assert torch.equal(p2v.cpu(), ref_p2v)
    torch.manual_seed(0)
    net = P.PointTransformerV3(in_channels=6, enc_depths=(1, 1, 1, 1, 1), dec_depths=(1, 1, 1, 1)).eval().cuda()
    with torch.inference_mode():
        torch.manual_seed(1)
        a = net(dict(data)).feat
        torch.manual_seed(1)
        b = net({"coord": coord[keep].cuda(), "grid_coord": ref_grid[keep].cuda(), "feat": feat[keep].cuda(),
                 "offset": ref_off.cuda(), "grid_size": 0.02}).feat
    assert torch.equal(a, b)
    # per-point results: scatter the voxel features back
    assert a[p2v].shape == (n, a.shape[1])
