"""Parity of every C-ABI operator with the CPU oracle on identical seeded
inputs: bit-exact for index work, within the stated tolerance for features."""
import pytest
import torch
import torch.nn.functional as F

from helpers import TOL, assert_close, rel_l2, small_batch
from oracle import ptv3_oracle as O
from pointtransformerv3_b200 import ops

pytestmark = pytest.mark.gpu
ORDERS = ["z", "z-trans", "hilbert", "hilbert-trans"]


@pytest.mark.parametrize("counts,K", [([5000], 1024), ([1024], 1024), ([1025], 1024), ([2048, 2049], 1024),
                                      ([300, 70, 4000], 128), ([70, 56], 56), ([10], 1024),
                                      ([999, 1, 3000], 1000)])
def test_pad_plan(counts, K):
    offset = torch.cumsum(torch.tensor(counts), 0)
    pad, unpad, cu = O.pad_plan(offset, K)
    gp, gu, gc = ops.pad_plan(offset.cuda(), counts, K)
    assert torch.equal(gp.cpu(), pad) and torch.equal(gu.cpu(), unpad) and torch.equal(gc.cpu(), cu)


def _attention_case(sizes, C, H, K, dtype, seed=0):
    data = small_batch(sizes, seed)
    offset = data["offset"]
    batch = O.offset_to_batch(offset)
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ["hilbert"])
    g = torch.Generator().manual_seed(seed)
    n = batch.shape[0]
    feat = torch.randn(n, C, generator=g)
    wq = torch.randn(3 * C, C, generator=g) / C ** 0.5
    bq = torch.randn(3 * C, generator=g) * 0.1
    wp = torch.randn(C, C, generator=g) / C ** 0.5
    bp = torch.randn(C, generator=g) * 0.1
    ref32 = O.attention(feat, wq, bq, wp, bp, order[0], inverse[0], offset, H, K)
    cast = lambda t: t.to(dtype)
    ref = O.attention(cast(feat), cast(wq), cast(bq), cast(wp), cast(bp), order[0], inverse[0], offset, H, K)
    counts = O.offset_to_counts(offset).tolist()
    Ke = min(min(counts), K)
    pad, unpad, cu = ops.pad_plan(offset.cuda(), counts, Ke)
    dev = lambda t: cast(t).cuda()
    qkv = F.linear(dev(feat), dev(wq), dev(bq))
    core = ops.attention(qkv, order[0].cuda(), pad, unpad, cu, H, Ke, (C // H) ** -0.5)
    got = F.linear(core, dev(wp), dev(bp))
    return got, ref, ref32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes,C,H,K", [([3000], 64, 4, 1024), ([1500, 700], 32, 2, 128),
                                         ([400, 90], 64, 4, 1024), ([2500], 128, 2, 512)])
def test_attention_matches_oracle(sizes, C, H, K, dtype):
    got, ref, ref32 = _attention_case(sizes, C, H, K, dtype)
    assert got.dtype == dtype
    assert_close(got, ref, what="attention", **TOL[dtype])
    if dtype == torch.bfloat16:
        # the kernel must be about as close to fp32 as the reference's own bf16 path
        assert rel_l2(got, ref32) <= 2.0 * rel_l2(ref, ref32) + 1e-3
    else:
        assert rel_l2(got, ref) < 1e-5


def test_kernel_map_matches_oracle_and_is_symmetric():
    data = small_batch([4000, 2500], 1)
    batch = O.offset_to_batch(data["offset"])
    ind = O.sparse_indices(batch, data["grid_coord"])
    for k in (3, 5):
        ref = O.kernel_map(ind, k)
        got = ops.kmap_build(ind.cuda(), k).cpu()
        assert torch.equal(got.t().long(), ref)
        kv = k ** 3
        n = ind.shape[0]
        ar = torch.arange(n)
        for o in range(kv):
            j = got[o].long()
            m = j >= 0
            assert torch.equal(got[kv - 1 - o][j[m]].long(), ar[m])
        assert torch.equal(got[kv // 2].long(), ar)


def test_kernel_map_duplicates_and_edges():
    ind = torch.tensor([[0, 0, 0, 0], [0, 1, 0, 0], [0, 0, 0, 0], [1, 0, 0, 0], [0, 65535, 65535, 65535]],
                       dtype=torch.int32)
    ref = O.kernel_map(ind, 3)
    got = ops.kmap_build(ind.cuda(), 3).cpu()
    assert torch.equal(got.t().long(), ref)


def test_batch_indices_match_torch():
    """ptv3_batch_indices against repeat_interleave and the concatenation it replaces (an empty
    scene in the middle, one scene, many scenes)."""
    from pointtransformerv3_b200.point import offset2batch
    g = torch.Generator().manual_seed(3)
    for counts in ([5, 0, 7, 1], [1000], [3] * 40, [0, 0, 9]):
        offset = torch.tensor(counts).cumsum(0)
        n = int(offset[-1])
        grid = torch.randint(0, 500, (n, 3), generator=g, dtype=torch.int32)
        batch, ind = ops.batch_indices(offset.cuda(), n, grid.cuda())
        want = offset2batch(offset, n)
        assert torch.equal(batch.cpu(), want)
        assert torch.equal(ind.cpu(), torch.cat([want.unsqueeze(-1).int(), grid], 1))


@pytest.mark.parametrize("k", [3, 5, 7])
def test_kmap_in_row_order(k):
    """ptv3_kmap_build_ordered: the table of the natural order with its columns permuted, bit for bit."""
    g = torch.Generator().manual_seed(k)
    ind = torch.unique(torch.cat([torch.randint(0, 2, (3000, 1), generator=g),
                                  torch.randint(0, 24, (3000, 3), generator=g)], 1), dim=0).int()
    order = torch.randperm(ind.shape[0], generator=g)
    plain = ops.kmap_build(ind.cuda(), k)
    got = ops.kmap_build(ind.cuda(), k, row_order=order.cuda())
    assert torch.equal(got, plain.index_select(1, order.cuda()))
    with pytest.raises(ValueError):
        ops.kmap_build(ind.cuda(), k, row_order=order[:-1].cuda())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("k,cin,cout", [(3, 32, 32), (3, 64, 64), (3, 128, 128), (5, 6, 32), (5, 4, 32),
                                        (3, 48, 80)])
def test_subm_conv_matches_oracle(k, cin, cout, dtype):
    data = small_batch([3000, 1200], 2)
    batch = O.offset_to_batch(data["offset"])
    ind = O.sparse_indices(batch, data["grid_coord"])
    n = ind.shape[0]
    g = torch.Generator().manual_seed(k * 1000 + cin)
    feat = torch.randn(n, cin, generator=g).to(dtype)
    w = (torch.randn(cout, k, k, k, cin, generator=g) / (k ** 3 * cin) ** 0.5 * 3).to(dtype)
    b = (torch.randn(cout, generator=g) * 0.1).to(dtype)
    nbr_ref = O.kernel_map(ind, k)
    ref = O.subm_conv(feat, nbr_ref, w, b)
    nbr = ops.kmap_build(ind.cuda(), k)
    got = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda())
    assert_close(got, ref, what="conv", **TOL[dtype])
    got_nb = ops.subm_conv(feat.cuda(), nbr, w.cuda(), None)
    assert_close(got_nb, O.subm_conv(feat, nbr_ref, w, None), what="conv no bias", **TOL[dtype])


@pytest.mark.parametrize("sizes", [[5000], [3000, 800, 1500]])
@pytest.mark.parametrize("perm", [None, [2, 0, 3, 1]])
def test_pool_plan_matches_oracle(sizes, perm):
    data = small_batch(sizes, 3)
    offset = data["offset"]
    batch = O.offset_to_batch(offset)
    fine_perm = torch.tensor([1, 3, 0, 2])
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ORDERS, perm=fine_perm)
    # walk three levels, feeding each level's oracle outputs to both sides
    grid, b = data["grid_coord"], batch
    for level in range(3):
        p = None if perm is None else torch.tensor(perm)
        ref = O.pooling_plan(code, depth, 2, p)
        got = ops.pool_plan(code.cuda(), order.cuda(), grid.cuda(), b.cuda(), len(sizes),
                            ref["pooling_depth"], perm)
        m = ref["code"].shape[1]
        assert got["m"] == m
        assert torch.equal(got["cluster"].cpu(), ref["cluster"])
        assert torch.equal(got["code"].cpu(), ref["code"])
        assert torch.equal(got["order"].cpu(), ref["order"])
        assert torch.equal(got["inverse"].cpu(), ref["inverse"])
        assert torch.equal(got["idx_ptr"].cpu(), ref["idx_ptr"])
        rg = grid[ref["head"]] >> ref["pooling_depth"]
        assert torch.equal(got["grid_coord"].cpu(), rg)
        rb = b[ref["head"]]
        assert torch.equal(got["batch"].cpu(), rb)
        assert got["counts"] == torch.bincount(rb, minlength=len(sizes)).tolist()
        # every head is a member of its cluster
        assert torch.equal(ref["cluster"][got["head"].cpu()], torch.arange(m))
        code, order, depth, grid, b = ref["code"], ref["order"], ref["depth"], rg, rb


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pool_and_unpool_features(dtype):
    data = small_batch([4000, 1000], 4)
    batch = O.offset_to_batch(data["offset"])
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ORDERS)
    plan = O.pooling_plan(code, depth, 2)
    n, C = batch.shape[0], 64
    g = torch.Generator().manual_seed(5)
    x = torch.randn(n, C, generator=g).to(dtype)
    sd = {"w": 1 + 0.1 * torch.randn(C, generator=g), "b": 0.1 * torch.randn(C, generator=g),
          "m": 0.1 * torch.randn(C, generator=g), "v": 0.5 + torch.rand(C, generator=g)}
    bn = lambda t: F.batch_norm(t, sd["m"].to(dtype), sd["v"].to(dtype), sd["w"].to(dtype), sd["b"].to(dtype),
                                False, 0.0, 1e-3)
    ref = F.gelu(bn(O.segment_reduce(x[plan["indices"]], plan["idx_ptr"], "max")))
    ref_coord = O.segment_reduce(data["coord"][plan["indices"]], plan["idx_ptr"], "mean")
    scale = (sd["w"] / torch.sqrt(sd["v"] + 1e-3)).cuda()
    shift = (sd["b"] - sd["m"] * sd["w"] / torch.sqrt(sd["v"] + 1e-3)).cuda()
    got, got_coord = ops.pool(x.cuda(), data["coord"].cuda(), order[0].cuda(), plan["idx_ptr"].cuda(), scale, shift)
    assert_close(got, ref, what="pool", **TOL[dtype])
    assert_close(got_coord, ref_coord, atol=1e-5, rtol=1e-5, what="coord mean")
    # unpool
    m = plan["code"].shape[1]
    child = torch.randn(m, C, generator=g).to(dtype)
    ref_a = F.gelu(bn(child))
    ref_b = F.gelu(bn(x))
    ref_u = ref_b + ref_a[plan["cluster"]]
    out, act = ops.unpool(x.cuda(), child.cuda(), plan["cluster"].cuda(), scale, shift, scale, shift)
    assert_close(out, ref_u, what="unpool", **TOL[dtype])
    assert_close(act, ref_b, what="unpool skip", **TOL[dtype])


@pytest.mark.parametrize("sizes,C,H,K", [([3000], 64, 4, 1024), ([1100, 90, 2049], 32, 2, 1024),
                                         ([5000], 128, 8, 2048), ([777], 16, 1, 100)])
def test_attention_tensor_core_path_matches_cuda_core_path(sizes, C, H, K):
    """Same inputs through both kernels (algo 2 vs algo 1), bf16."""
    data = small_batch(sizes, 7)
    offset = data["offset"]
    counts = O.offset_to_counts(offset).tolist()
    batch = O.offset_to_batch(offset)
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ["z-trans"])
    g = torch.Generator().manual_seed(1)
    qkv = (torch.randn(batch.shape[0], 3 * C, generator=g) * 1.5).bfloat16().cuda()
    Ke = min(min(counts), K)
    pad, unpad, cu = ops.pad_plan(offset.cuda(), counts, Ke)
    a = ops.attention(qkv, order[0].cuda(), pad, unpad, cu, H, Ke, (C // H) ** -0.5, algo=1)
    b = ops.attention(qkv, order[0].cuda(), pad, unpad, cu, H, Ke, (C // H) ** -0.5, algo=2)
    assert_close(b, a, atol=1e-2, rtol=1e-2, what="tensor-core vs CUDA-core attention")
    assert rel_l2(b, a) < 5e-3


@pytest.mark.parametrize("sizes,C,H,K", [([3000], 64, 4, 1024), ([1100, 90, 2049], 32, 2, 1024),
                                         ([5000], 128, 8, 512), ([777], 16, 1, 100), ([130, 129, 128, 127], 32, 2, 1024),
                                         ([2048, 1025], 64, 4, 1024), ([300], 512, 32, 1024)])
def test_attention_tcgen05_path_matches_cuda_core_path(sizes, C, H, K):
    """Same inputs through the tcgen05 kernel (algo 4) and the CUDA-core kernel
    (algo 1), bf16: full and ragged patches, patches shorter than a key block,
    borrowed rows of a last patch."""
    data = small_batch(sizes, 11)
    offset = data["offset"]
    counts = O.offset_to_counts(offset).tolist()
    batch = O.offset_to_batch(offset)
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ["hilbert-trans"])
    g = torch.Generator().manual_seed(2)
    qkv = (torch.randn(batch.shape[0], 3 * C, generator=g) * 1.5).bfloat16().cuda()
    # flash semantics (patch size kept, short scenes are one short patch) and the
    # non-flash rule (patch shrunk to the smallest scene)
    for Ke in (K, min(min(counts), K)):
        pad, unpad, cu = ops.pad_plan(offset.cuda(), counts, Ke)
        a = ops.attention(qkv, order[0].cuda(), pad, unpad, cu, H, Ke, (C // H) ** -0.5, algo=1)
        b = ops.attention(qkv, order[0].cuda(), pad, unpad, cu, H, Ke, (C // H) ** -0.5, algo=4)
        assert_close(b, a, atol=1e-2, rtol=1e-2, what="tcgen05 vs CUDA-core attention")
        assert rel_l2(b, a) < 5e-3


def test_attention_tcgen05_large_scores():
    """Scores far from zero (|s| up to a few hundred): the running maximum and the
    rescaling of the output across key blocks must hold."""
    n, C, H, K = 4096, 32, 2, 1024
    g = torch.Generator().manual_seed(5)
    grid = torch.randint(0, 64, (n, 3), generator=g, dtype=torch.int32)
    order = O.serialization(grid, torch.zeros(n, dtype=torch.int64), ["z"])[1]
    qkv = torch.randn(n, 3 * C, generator=g)
    qkv[:, :2 * C] *= 6.0
    qkv = qkv.bfloat16().cuda()
    pad, unpad, cu = ops.pad_plan(torch.tensor([n]).cuda(), [n], K)
    a = ops.attention(qkv, order[0].cuda(), pad, unpad, cu, H, K, 0.25, algo=1)
    b = ops.attention(qkv, order[0].cuda(), pad, unpad, cu, H, K, 0.25, algo=4)
    assert bool(torch.isfinite(b.float()).all())
    assert rel_l2(b, a) < 1e-2


@pytest.mark.parametrize("algo,dtype", [(0, torch.bfloat16), (1, torch.bfloat16), (1, torch.float32),
                                        (4, torch.bfloat16)])
def test_attention_reports_a_patch_longer_than_max_seqlen(algo, dtype):
    """A plan made for patches of 512 rows handed to a call that states max_seqlen = 128
    (what a cached plan of another patch size amounts to): every path skips the long
    patches and reports PTV3_STATUS_BAD_INDEX through the status word; nothing is read
    or written out of bounds."""
    from pointtransformerv3_b200 import _lib
    n, C, H = 3000, 64, 4
    g = torch.Generator().manual_seed(0)
    qkv = torch.randn(n, 3 * C, generator=g).to(dtype).cuda()
    order = torch.randperm(n, generator=g).cuda()
    pad, unpad, cu = ops.pad_plan(torch.tensor([n]).cuda(), [n], 512)
    st = ops.new_status(qkv.device)
    ops.attention(qkv, order, pad, unpad, cu, H, 128, 0.25, algo=algo, status=st)
    assert int(st.item()) & 1, "status word 0x%x" % int(st.item())
    with pytest.raises(_lib.Ptv3Error):
        ops.attention(qkv, order, pad, unpad, cu, H, 128, 0.25, algo=algo)
    # the same plan with the right max_seqlen is clean
    st.zero_()
    ops.attention(qkv, order, pad, unpad, cu, H, 512, 0.25, algo=algo, status=st)
    assert int(st.item()) == 0


@pytest.mark.parametrize("ALGO", [2, 4])
def test_attention_config2_size_bf16(ALGO):
    """N = 120 000, C = 64, 4 heads, patch 1024 (118 patches, the last one padded by
    borrowing): both tensor-core paths against the fp32 oracle on a row sample."""
    n, C, H, K = 120_000, 64, 4, 1024
    g = torch.Generator().manual_seed(0)
    grid = torch.randint(0, 512, (n, 3), generator=g, dtype=torch.int32)
    batch = torch.zeros(n, dtype=torch.int64)
    offset = torch.tensor([n])
    code, order, inverse, depth = O.serialization(grid, batch, ["hilbert"])
    qkv = torch.randn(n, 3 * C, generator=g)
    pad, unpad, cu = ops.pad_plan(offset.cuda(), [n], K)
    assert pad.numel() == 120_832 and cu.numel() == 119
    got = ops.attention(qkv.bfloat16().cuda(), order[0].cuda(), pad, unpad, cu, H, K, 0.25, algo=ALGO).float().cpu()
    # oracle for the first, a middle and the (borrowing) last patch
    rp, ru, rc = O.pad_plan(offset, K)
    x = qkv.bfloat16().float()
    for patch in (0, 57, 117):
        rows = order[0][rp[patch * K:(patch + 1) * K]]
        q, k, v = x[rows].reshape(K, 3, H, 16).permute(1, 2, 0, 3)
        w = torch.softmax((q * 0.25) @ k.transpose(-1, -2), -1)
        ref = (w @ v).transpose(0, 1).reshape(K, C)
        own = ru[inverse[0][rows]] == torch.arange(patch * K, (patch + 1) * K)
        assert_close(got[rows[own]], ref[own], atol=2e-2, rtol=1e-2, what="patch %d" % patch)
        assert rel_l2(got[rows[own]], ref[own]) < 1e-2


@pytest.mark.parametrize("c", [32, 64, 128, 256])
@pytest.mark.parametrize("permuted", [False, True])
def test_subm_conv_tensor_core_path(c, permuted):
    """bf16 tensor-core convolution against the fp32 oracle and the CUDA-core path,
    with and without a space-filling-curve tile order."""
    data = small_batch([6000, 2500], 8)
    batch = O.offset_to_batch(data["offset"])
    ind = O.sparse_indices(batch, data["grid_coord"])
    n = ind.shape[0]
    g = torch.Generator().manual_seed(c)
    feat = torch.randn(n, c, generator=g).bfloat16()
    w = (torch.randn(c, 3, 3, 3, c, generator=g) / (9 * c) ** 0.5).bfloat16()
    b = (torch.randn(c, generator=g) * 0.1).bfloat16()
    ref = O.subm_conv(feat.float(), O.kernel_map(ind, 3), w.float(), b.float())
    nbr = ops.kmap_build(ind.cuda(), 3)
    row_order = None
    if permuted:
        code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ["z"])
        row_order = order[0].cuda()
        nbr = nbr.index_select(1, row_order)
    got = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda(), algo=2, row_order=row_order)
    base = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda(), algo=1, row_order=row_order)
    assert_close(got, ref, what="tensor-core conv vs fp32 oracle", **TOL[torch.bfloat16])
    assert_close(got, base, atol=1e-2, rtol=1e-2, what="tensor-core vs CUDA-core conv")
    assert rel_l2(got, ref) < 4e-3


@pytest.mark.parametrize("voxels,cin,cout", [(28000, 256, 256), (14000, 256, 512)])
def test_subm_conv_tcgen05_wide_tiles(voxels, cin, cout):
    """Inputs long and wide enough for the 256-output-channel tiles of the tcgen05 convolution
    (at least 148 of them): against the fp32 oracle and the mma.sync path, in serialized row order,
    twice for bit-identical results."""
    data = small_batch([voxels * 7 // 10, voxels * 3 // 10], 9)
    batch = O.offset_to_batch(data["offset"])
    ind = torch.unique(O.sparse_indices(batch, data["grid_coord"]), dim=0)
    n = ind.shape[0]
    assert (n + 127) // 128 * (cout // 256) >= 148
    g = torch.Generator().manual_seed(voxels + cout)
    feat = torch.randn(n, cin, generator=g).bfloat16()
    w = (torch.randn(cout, 3, 3, 3, cin, generator=g) / (9 * cin) ** 0.5).bfloat16()
    b = (torch.randn(cout, generator=g) * 0.1).bfloat16()
    ref = O.subm_conv(feat.float(), O.kernel_map(ind, 3), w.float(), b.float())
    code, order, inverse, depth = O.serialization(ind[:, 1:], ind[:, 0].long(), ["z"])
    row_order = order[0].cuda()
    nbr = ops.kmap_build(ind.cuda(), 3, row_order=row_order)
    got = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda(), algo=3, row_order=row_order)
    again = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda(), algo=3, row_order=row_order)
    assert torch.equal(got, again)
    assert_close(got, ref, what="tcgen05 conv (256-wide tiles) vs fp32 oracle", **TOL[torch.bfloat16])
    assert rel_l2(got, ref) < 4e-3
    base = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda(), algo=2, row_order=row_order)
    assert_close(got, base, atol=1e-2, rtol=1e-2, what="tcgen05 vs mma.sync conv")


@pytest.mark.parametrize("permuted", [False, True])
@pytest.mark.parametrize("cin,cout,shift", [(32, 32, 0), (64, 64, 0), (128, 128, 1), (256, 256, 2), (512, 512, 3),
                                            (64, 192, 1)])
def test_subm_conv_tcgen05_path(cin, cout, shift, permuted):
    """bf16 convolution with the accumulator in tensor memory against the fp32 oracle and the
    mma.sync path, on a fine level and on coarsened ones (denser neighbourhoods), sizes that are not
    multiples of the tile, and twice for bit-identical results."""
    data = small_batch([6000, 2500], 8 + shift)
    batch = O.offset_to_batch(data["offset"])
    ind = O.sparse_indices(batch, data["grid_coord"] >> shift)
    ind = torch.unique(ind, dim=0)
    n = ind.shape[0]
    g = torch.Generator().manual_seed(cin + cout)
    feat = torch.randn(n, cin, generator=g).bfloat16()
    w = (torch.randn(cout, 3, 3, 3, cin, generator=g) / (9 * cin) ** 0.5).bfloat16()
    b = (torch.randn(cout, generator=g) * 0.1).bfloat16()
    ref = O.subm_conv(feat.float(), O.kernel_map(ind, 3), w.float(), b.float())
    nbr = ops.kmap_build(ind.cuda(), 3)
    row_order = None
    if permuted:
        code, order, inverse, depth = O.serialization(ind[:, 1:], ind[:, 0].long(), ["z"])
        row_order = order[0].cuda()
        nbr = nbr.index_select(1, row_order)
    got = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda(), algo=3, row_order=row_order)
    again = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda(), algo=3, row_order=row_order)
    assert torch.equal(got, again)
    assert_close(got, ref, what="tcgen05 conv vs fp32 oracle", **TOL[torch.bfloat16])
    assert rel_l2(got, ref) < 4e-3
    if cin == cout:
        base = ops.subm_conv(feat.cuda(), nbr, w.cuda(), b.cuda(), algo=2, row_order=row_order)
        assert_close(got, base, atol=1e-2, rtol=1e-2, what="tcgen05 vs mma.sync conv")
    nb = ops.subm_conv(feat.cuda(), nbr, w.cuda(), None, algo=3, row_order=row_order)
    assert_close(nb, O.subm_conv(feat.float(), O.kernel_map(ind, 3), w.float(), None), what="no bias",
                 **TOL[torch.bfloat16])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C", [32, 48, 64, 128, 256, 512])
def test_add_layernorm(C, dtype):
    n = 3001
    g = torch.Generator().manual_seed(C)
    x = torch.randn(n, C, generator=g).to(dtype)
    r = torch.randn(n, C, generator=g).to(dtype)
    ln1 = torch.nn.LayerNorm(C)
    ln2 = torch.nn.LayerNorm(C)
    for ln in (ln1, ln2):
        ln.weight.data = 1 + 0.1 * torch.randn(C, generator=g)
        ln.bias.data = 0.1 * torch.randn(C, generator=g)
    ln1, ln2 = ln1.to(dtype), ln2.to(dtype)
    ref_s = r + ln1(x)
    ref_y = ln2(ref_s)
    import copy
    c1, c2 = copy.deepcopy(ln1).cuda(), copy.deepcopy(ln2).cuda()
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    s, y = ops.add_layernorm(x.cuda(), r.cuda(), c1, c2)
    assert_close(s, ref_s, what="sum", **tol)
    assert_close(y, ref_y, what="norm", **tol)
    s, y = ops.add_layernorm(x.cuda(), r.cuda(), None, c2)
    assert_close(s, r + x, what="plain sum", **tol)
    assert_close(y, ln2(r + x), what="norm of plain sum", **tol)
    s, y = ops.add_layernorm(x.cuda(), None, c1, None)
    assert y is None
    assert_close(s, ln1(x), what="plain layer norm", **tol)
    s, y = ops.add_layernorm(x.cuda(), r.cuda(), None, None)
    assert_close(s, r + x, what="add only", **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cin,cout,k,fuse", [(6, 32, 5, True), (4, 32, 5, False), (3, 16, 3, True), (8, 64, 3, False)])
def test_subm_conv_direct(cin, cout, k, fuse, dtype):
    data = small_batch([3000, 1200], 12)
    batch = O.offset_to_batch(data["offset"])
    ind = O.sparse_indices(batch, data["grid_coord"])
    n = ind.shape[0]
    g = torch.Generator().manual_seed(cin * 100 + cout)
    feat = torch.randn(n, cin, generator=g).to(dtype)
    w = (torch.randn(cout, k, k, k, cin, generator=g) / (k ** 3 * cin) ** 0.5 * 3).to(dtype)
    ref = O.subm_conv(feat, O.kernel_map(ind, k), w, None)
    scale = shift = None
    if fuse:
        scale = (1 + 0.1 * torch.randn(cout, generator=g))
        shift = 0.1 * torch.randn(cout, generator=g)
        ref = F.gelu((ref.float() * scale + shift).to(dtype))
        scale, shift = scale.cuda(), shift.cuda()
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ["hilbert"])
    for row_order in (None, order[0].cuda()):
        got = ops.subm_conv_direct(feat.cuda(), ind.cuda(), w.cuda(), None, scale, shift, fuse, row_order)
        assert_close(got, ref, what="direct conv", **TOL[dtype])


@pytest.mark.parametrize("C", [32, 64])
@pytest.mark.parametrize("n", [128, 1000, 40_000])
def test_fused_mlp_tcgen05(C, n):
    """out = residual + fc2(GELU(fc1(x))) on the tcgen05 path against torch on CPU."""
    g = torch.Generator().manual_seed(C + n)
    x = torch.randn(n, C, generator=g).bfloat16()
    res = torch.randn(n, C, generator=g).bfloat16()
    w1 = (torch.randn(4 * C, C, generator=g) / C ** 0.5).bfloat16()
    b1 = (0.1 * torch.randn(4 * C, generator=g)).bfloat16()
    w2 = (torch.randn(C, 4 * C, generator=g) / (4 * C) ** 0.5).bfloat16()
    b2 = (0.1 * torch.randn(C, generator=g)).bfloat16()
    ref = res + F.linear(F.gelu(F.linear(x, w1, b1)), w2, b2)
    ref32 = res.float() + F.linear(F.gelu(F.linear(x.float(), w1.float(), b1.float())), w2.float(), b2.float())
    assert ops.mlp_supported(C, 4 * C, torch.bfloat16)
    got = ops.mlp(x.cuda(), w1.cuda(), b1.cuda(), w2.cuda(), b2.cuda(), res.cuda())
    assert_close(got, ref, what="fused mlp", **TOL[torch.bfloat16])
    assert rel_l2(got, ref32) <= 1.5 * rel_l2(ref, ref32) + 1e-3


@pytest.mark.parametrize("c", [128, 256])
@pytest.mark.parametrize("permuted", [False, True])
def test_subm_conv_pair_list_path(c, permuted):
    """Pair-list convolution (atomic fp32 accumulation) against the fp32 oracle, and
    the structure of the pair list itself."""
    data = small_batch([2000, 900], 14)
    batch = O.offset_to_batch(data["offset"])
    ind = O.sparse_indices(batch, data["grid_coord"] >> 2)
    ind = torch.unique(ind, dim=0)
    n = ind.shape[0]
    g = torch.Generator().manual_seed(c)
    feat = torch.randn(n, c, generator=g).bfloat16()
    w = (torch.randn(c, 3, 3, 3, c, generator=g) / (9 * c) ** 0.5).bfloat16()
    b = (torch.randn(c, generator=g) * 0.1).bfloat16()
    ref_nbr = O.kernel_map(ind, 3)
    ref = O.subm_conv(feat.float(), ref_nbr, w.float(), b.float())
    nbr = ops.kmap_build(ind.cuda(), 3)
    row_order = None
    if permuted:
        code, order, inverse, depth = O.serialization(ind[:, 1:], ind[:, 0].long(), ["z"])
        row_order = order[0].cuda()
        nbr = nbr.index_select(1, row_order)
    pairs = ops.conv_pairs_build(nbr, row_order)
    off = pairs["off_start"].cpu().tolist()
    tiles = pairs["tile_start"].cpu().tolist()
    counts = (ref_nbr >= 0).sum(0).tolist()
    assert [off[i + 1] - off[i] for i in range(27)] == counts
    assert [tiles[i + 1] - tiles[i] for i in range(27)] == [(c_ + 127) // 128 for c_ in counts]
    pin, pout = pairs["pair_in"].cpu()[: off[27]].long(), pairs["pair_out"].cpu()[: off[27]].long()
    for o in (0, 13, 26):
        sl = slice(off[o], off[o + 1])
        assert torch.equal(ref_nbr[pout[sl], o], pin[sl])
    got = ops.subm_conv_pairs(feat.cuda(), pairs, w.cuda(), b.cuda())
    assert_close(got, ref, what="pair-list conv", **TOL[torch.bfloat16])
    assert rel_l2(got, ref) < 4e-3


@pytest.mark.parametrize("k,n_out", [(32, 96), (64, 192), (128, 384), (64, 64), (32, 32), (128, 128), (128, 256)])
@pytest.mark.parametrize("n", [100, 5000])
def test_linear_tcgen05(k, n_out, n):
    g = torch.Generator().manual_seed(k + n_out + n)
    x = torch.randn(n, k, generator=g).bfloat16()
    w = (torch.randn(n_out, k, generator=g) / k ** 0.5).bfloat16()
    b = (0.1 * torch.randn(n_out, generator=g)).bfloat16()
    assert ops.linear_supported(k, n_out, False, torch.bfloat16)
    got = ops.linear(x.cuda(), w.cuda(), b.cuda())
    assert_close(got, F.linear(x, w, b), what="linear", **TOL[torch.bfloat16])
    assert rel_l2(got, F.linear(x.float(), w.float(), b.float())) < 5e-3


@pytest.mark.parametrize("n,k,n_out,gelu,res", [(3000, 256, 768, False, False), (2111, 256, 256, False, True),
                                                 (7000, 128, 512, True, False), (7000, 512, 128, False, True),
                                                 (500, 512, 1536, False, False), (129, 2048, 512, False, True),
                                                 (1, 64, 128, True, True), (2049, 1024, 256, False, False),
                                                 # long inputs: several tiles per CTA
                                                 (76801, 256, 256, False, True), (40000, 128, 512, True, False),
                                                 (50000, 256, 768, False, False), (90000, 512, 128, False, True),
                                                 # 128-column tiles with the weights resident; both epilogue steps
                                                 (70000, 128, 384, False, True), (60000, 64, 128, True, True)])
def test_gemm_tcgen05(n, k, n_out, gelu, res):
    """The streamed-weight Linear kernel against torch on CPU with the same roundings (GEMM result
    rounded to bf16, then GELU / residual sum rounded again)."""
    g = torch.Generator().manual_seed(n + k + n_out)
    x = torch.randn(n, k, generator=g).bfloat16()
    w = (torch.randn(n_out, k, generator=g) / k ** 0.5).bfloat16()
    b = (0.1 * torch.randn(n_out, generator=g)).bfloat16()
    r = torch.randn(n, n_out, generator=g).bfloat16() if res else None
    assert ops.gemm_supported(k, n_out, torch.bfloat16)
    got = ops.gemm(x.cuda(), w.cuda(), b.cuda(), None if r is None else r.cuda(), gelu)
    ref32 = F.linear(x.float(), w.float(), b.float())
    ref = ref32.bfloat16()
    if gelu:
        ref = F.gelu(ref.float()).bfloat16()
        ref32 = F.gelu(ref32)
    if res:
        ref = (ref.float() + r.float()).bfloat16()
        ref32 = ref32 + r.float()
    assert_close(got, ref, what="gemm", **TOL[torch.bfloat16])
    assert rel_l2(got, ref32) < 5e-3
    # without a bias
    got = ops.gemm(x.cuda(), w.cuda(), None, None, False)
    assert_close(got, F.linear(x.float(), w.float()).bfloat16(), what="gemm without bias", **TOL[torch.bfloat16])


def test_gemm_rejects_unsupported_shapes():
    from pointtransformerv3_b200 import _lib
    x = torch.zeros(10, 96, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 96, dtype=torch.bfloat16, device="cuda")
    assert not ops.gemm_supported(96, 128, torch.bfloat16)
    with pytest.raises(_lib.Ptv3Error):
        ops.gemm(x, w)


@pytest.mark.parametrize("C", [32, 64, 128])
@pytest.mark.parametrize("with_ln1", [True, False])
def test_linear_ln_tcgen05(C, with_ln1):
    n = 3000
    g = torch.Generator().manual_seed(C * 2 + with_ln1)
    x = torch.randn(n, C, generator=g).bfloat16()
    res = (torch.randn(n, C, generator=g) * 2 + 0.5).bfloat16()
    w = (torch.randn(C, C, generator=g) / C ** 0.5).bfloat16()
    b = (0.1 * torch.randn(C, generator=g)).bfloat16()
    ln1, ln2 = torch.nn.LayerNorm(C), torch.nn.LayerNorm(C)
    for ln in (ln1, ln2):
        ln.weight.data = 1 + 0.1 * torch.randn(C, generator=g)
        ln.bias.data = 0.1 * torch.randn(C, generator=g)
    ln1, ln2 = ln1.bfloat16(), ln2.bfloat16()
    y = F.linear(x, w, b)
    ref_s = res + (ln1(y) if with_ln1 else y)
    ref_n = ln2(ref_s)
    import copy
    c1, c2 = copy.deepcopy(ln1).cuda(), copy.deepcopy(ln2).cuda()
    s, nrm = ops.linear_ln(x.cuda(), w.cuda(), b.cuda(), res.cuda(), c1 if with_ln1 else None, c2)
    assert_close(s, ref_s, what="sum", **TOL[torch.bfloat16])
    assert_close(nrm, ref_n, what="norm", **TOL[torch.bfloat16])
    # against fp32 arithmetic: as close as the bf16 reference sequence is
    y32 = F.linear(x.float(), w.float(), b.float())
    s32 = res.float() + (F.layer_norm(y32, (C,), ln1.weight.float(), ln1.bias.float()) if with_ln1 else y32)
    n32 = F.layer_norm(s32, (C,), ln2.weight.float(), ln2.bias.float())
    assert rel_l2(nrm, n32) <= 1.5 * rel_l2(ref_n, n32) + 1e-3


@pytest.mark.parametrize("reduce", ["max", "min", "sum", "mean"])
def test_pool_reduce_modes(reduce):
    """All four reductions of SerializedPooling (model.py:626, 684-686)."""
    data = small_batch([3000, 800], 15)
    batch = O.offset_to_batch(data["offset"])
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ORDERS)
    plan = O.pooling_plan(code, depth, 2)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(batch.shape[0], 32, generator=g)
    ref = O.segment_reduce(x[plan["indices"]], plan["idx_ptr"], reduce)
    got, _ = ops.pool(x.cuda(), None, order[0].cuda(), plan["idx_ptr"].cuda(), None, None, reduce)
    assert_close(got, ref, atol=1e-5, rtol=1e-5, what="pool " + reduce)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,C,K", [(1, 64, 13), (5000, 64, 20), (70_000, 64, 13), (3000, 32, 40), (2000, 128, 64)])
def test_seg_head_matches_torch(n, C, K, dtype):
    """Linear + arg max in one pass against F.linear / argmax (fp32 accumulation on both
    sides; labels must agree wherever the two best logits are not within rounding)."""
    g = torch.Generator().manual_seed(n + K)
    feat = torch.randn(n, C, generator=g).to(dtype)
    w = (torch.randn(K, C, generator=g) / C ** 0.5).to(dtype)
    b = (torch.randn(K, generator=g) * 0.1).to(dtype)
    ref = F.linear(feat.float(), w.float(), b.float())
    logits, labels = ops.seg_head(feat.cuda(), w.cuda(), b.cuda())
    assert logits.dtype == dtype and labels.dtype == torch.int64
    assert_close(logits, ref.to(dtype), what="seg head logits", **TOL[dtype])
    # arg max of exactly what was returned, lowest index on ties
    assert torch.equal(labels.cpu(), logits.float().cpu().argmax(1))
    top2 = ref.topk(2, dim=1).values
    clear = (top2[:, 0] - top2[:, 1]) > (1e-4 if dtype == torch.float32 else 5e-2)
    assert torch.equal(labels.cpu()[clear], ref.argmax(1)[clear])
    only_labels = ops.seg_head(feat.cuda(), w.cuda(), b.cuda(), want_logits=False)
    assert only_labels[0] is None and torch.equal(only_labels[1], labels)
