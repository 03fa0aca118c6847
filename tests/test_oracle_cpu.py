"""Pins the CPU oracle: against the committed golden vectors (generated from
the unmodified reference by tests/golden/make_golden.py) and, where the
reference tree is present, against the reference executed live."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from helpers import small_batch
from oracle import cenc, ptv3_oracle as O, refload, weights

ORDERS = ["z", "z-trans", "hilbert", "hilbert-trans"]
SMALL_CFG = dict(enc_depths=(1, 1, 1, 2, 1), enc_channels=(32, 32, 64, 64, 128), enc_num_head=(2, 2, 4, 4, 8),
                 enc_patch_size=(128,) * 5, dec_depths=(1, 1, 1, 1), dec_channels=(32, 32, 64, 64),
                 dec_num_head=(2, 2, 4, 4), dec_patch_size=(128,) * 4)


def load(name):
    return np.load(os.path.join(GOLDEN, name))


def from_bf16_bits(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def test_encode_golden():
    g = load("serialization.npz")
    for depth in (1, 3, 9, 11, 16):
        for o in ORDERS:
            got = cenc.encode(g[f"grid_d{depth}"], g[f"batch_d{depth}"], depth, o)
            assert (got == g[f"code_d{depth}_{o}"]).all(), (depth, o)


def test_point_serialization_golden():
    g = load("serialization.npz")
    data = small_batch([3000, 1700], seed=11)
    batch = O.offset_to_batch(data["offset"])
    torch.manual_seed(5)
    perm = torch.randperm(4)
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ORDERS, perm=perm)
    assert depth == int(g["point_depth"])
    assert (code.numpy() == g["point_code"]).all()
    assert (order.numpy() == g["point_order"]).all()
    assert (inverse.numpy() == g["point_inverse"]).all()


def test_encode_properties():
    rng = np.random.default_rng(0)
    for depth in (2, 7, 16):
        g = rng.integers(0, 1 << depth, size=(4000, 3)).astype(np.int32)
        for o in ORDERS:
            c = cenc.encode(g, None, depth, o)
            # hierarchical: dropping one level == encoding the parent cell
            assert (c >> 3 == cenc.encode(g >> 1, None, depth - 1, o)).all() if depth > 1 else True
            # injective on distinct cells
            key = (g[:, 0].astype(np.int64) << 40) | (g[:, 1].astype(np.int64) << 20) | g[:, 2]
            assert len(np.unique(c)) == len(np.unique(key))


def test_edge_sizes():
    assert cenc.encode(np.zeros((0, 3), np.int32), None, 16, "hilbert").shape == (0,)
    assert cenc.argsort_stable(np.zeros(0, np.int64)).shape == (0,)
    one = cenc.encode(np.array([[5, 6, 7]], np.int32), np.array([3]), 16, "z")
    assert one.shape == (1,) and one[0] >> 48 == 3


def _attention_oracle(name, sizes, C, H, K, order_index, dtype):
    data = small_batch(sizes, seed=21)
    batch = O.offset_to_batch(data["offset"])
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ["hilbert", "z"])
    n = batch.shape[0]
    feat = weights.keyed_tensor("attention.feat." + name, (n, C)).to(dtype)
    lin = lambda k, shape, fan: weights.keyed_tensor("attention.%s.%s" % (name, k), shape)
    sd = {
        "qkv.weight": lin("qkv.weight", (3 * C, C), C) / C ** 0.5,
        "qkv.bias": 0.1 * lin("qkv.bias", (3 * C,), C),
        "proj.weight": lin("proj.weight", (C, C), C) / C ** 0.5,
        "proj.bias": 0.1 * lin("proj.bias", (C,), C),
    }
    sd = {k: v.to(dtype) for k, v in sd.items()}
    return O.attention(feat, sd["qkv.weight"], sd["qkv.bias"], sd["proj.weight"], sd["proj.bias"],
                       order[order_index], inverse[order_index], data["offset"], H, K), data


@pytest.mark.parametrize("name,sizes,C,H,K,oi", [("a", [1800], 32, 2, 128, 0), ("b", [700, 90, 400], 64, 4, 256, 1)])
def test_attention_golden(name, sizes, C, H, K, oi):
    g = load("attention.npz")
    got, data = _attention_oracle(name, sizes, C, H, K, oi, torch.float32)
    assert np.abs(got.numpy() - g[name + "_fp32"]).max() < 1e-5
    got16, _ = _attention_oracle(name, sizes, C, H, K, oi, torch.bfloat16)
    ref16 = from_bf16_bits(g[name + "_bf16"]).float()
    assert (got16.float() - ref16).abs().max() < 2e-2
    counts = O.offset_to_counts(data["offset"]).tolist()
    pad, unpad, cu = O.pad_plan(data["offset"], min(min(counts), K))
    assert (pad.numpy() == g[name + "_pad"]).all() and (unpad.numpy() == g[name + "_unpad"]).all()
    assert (cu.numpy() == g[name + "_cu"]).all()


def test_pooling_golden():
    g = load("pooling.npz")
    data = small_batch([2500, 1200], seed=31)
    batch = O.offset_to_batch(data["offset"])
    torch.manual_seed(9)
    perm = torch.randperm(4)
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ORDERS, perm=perm)
    lv = O.Level(coord=data["coord"], grid_coord=data["grid_coord"], batch=batch, offset=data["offset"],
                 code=code, order=order, inverse=inverse, depth=depth, cluster=None, parent=None)
    n = batch.shape[0]
    feat = weights.keyed_tensor("pooling.feat", (n, 32))
    bn = lambda c: torch.nn.BatchNorm1d(c, eps=1e-3, momentum=0.01)

    class Down(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = torch.nn.Linear(32, 64)
            self.norm = torch.nn.Sequential(bn(64))

    class Up(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = torch.nn.Sequential(torch.nn.Linear(64, 48), bn(48))
            self.proj_skip = torch.nn.Sequential(torch.nn.Linear(32, 48), bn(48))

    sd = {"down." + k: v for k, v in weights.fill_state_dict(Down(), prefix="pooling.down.").items()}
    sd.update({"up." + k: v for k, v in weights.fill_state_dict(Up(), prefix="pooling.up.").items()})
    new, x = O.pool(sd, "down.", lv, feat, 2, True)
    assert np.abs(x.numpy() - g["down_feat"]).max() < 1e-5
    assert np.abs(new.coord.numpy() - g["down_coord"]).max() < 1e-5
    for k, v in (("grid_coord", new.grid_coord), ("batch", new.batch), ("serialized_code", new.code),
                 ("serialized_order", new.order), ("serialized_inverse", new.inverse),
                 ("pooling_inverse", new.cluster), ("offset", new.offset)):
        assert (v.numpy() == g["down_" + k]).all(), k
    assert new.depth == int(g["down_depth"])
    up, stale = O.unpool(sd, "up.", new, x, feat)
    assert np.abs(up.numpy() - g["up_feat"]).max() < 1e-5
    assert np.abs(stale.numpy() - g["up_sparse_feat"]).max() < 1e-5


def _oracle_state_dict(dtype=torch.float32):
    """The keyed fill needs the parameter names and shapes only; build them from
    the shipped module (host-side construction, no CUDA involved)."""
    from pointtransformerv3_b200 import PointTransformerV3
    net = PointTransformerV3(in_channels=6, enable_flash=False, **SMALL_CFG)
    sd = weights.fill_state_dict(net, prefix="ptv3.")
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}


def test_backbone_golden_fp32():
    g = load("backbone.npz")
    data = small_batch([6000, 4000], seed=41)
    sd = _oracle_state_dict()
    torch.manual_seed(1)
    out = O.ptv3_forward(sd, data, SMALL_CFG)
    assert np.abs(out.numpy() - g["fp32"]).max() < 1e-4


def test_backbone_golden_bf16():
    g = load("backbone.npz")
    data = small_batch([6000, 4000], seed=41)
    data["feat"] = data["feat"].bfloat16()
    sd = _oracle_state_dict(torch.bfloat16)
    torch.manual_seed(1)
    out = O.ptv3_forward(sd, data, SMALL_CFG)
    ref = from_bf16_bits(g["bf16"]).float()
    # same arithmetic in the same order: equal up to rare one-ulp reordering effects
    assert (out.float() - ref).abs().max() < 5e-2
    assert ((out.float() - ref).abs() > 1e-2).float().mean() < 1e-3


def test_subm_conv_against_dense_conv3d():
    """Pins the convolution convention: dense conv3d evaluated at the active sites."""
    g = torch.Generator().manual_seed(0)
    for k in (3, 5):
        B, S, cin, cout = 2, 9, 5, 7
        occ = torch.rand(B, S, S, S, generator=g) < 0.3
        idx = occ.nonzero().int()
        idx = idx[torch.randperm(idx.shape[0], generator=g)]
        feat = torch.randn(idx.shape[0], cin, generator=g)
        w = torch.randn(cout, k, k, k, cin, generator=g)
        bias = torch.randn(cout, generator=g)
        dense = torch.zeros(B, cin, S, S, S)
        dense[idx[:, 0].long(), :, idx[:, 1].long(), idx[:, 2].long(), idx[:, 3].long()] = feat
        ref = torch.nn.functional.conv3d(dense, w.permute(0, 4, 1, 2, 3), bias, padding=k // 2)
        ref = ref[idx[:, 0].long(), :, idx[:, 1].long(), idx[:, 2].long(), idx[:, 3].long()]
        got = O.subm_conv(feat, O.kernel_map(idx, k), w, bias)
        assert (got - ref).abs().max() < 1e-4


needs_ref = pytest.mark.skipif(refload.load_serialization() is None, reason="reference tree not present")


@needs_ref
def test_encode_vs_reference_live():
    ref = refload.load_serialization()
    rng = np.random.default_rng(3)
    for depth in range(1, 17):
        g = rng.integers(-5, (1 << depth) + 5, size=(800, 3)).astype(np.int32)
        b = rng.integers(0, 9, size=800)
        for o in ORDERS:
            r = ref.encode(torch.from_numpy(g), torch.from_numpy(b), depth, o).numpy()
            assert (r == cenc.encode(g, b, depth, o)).all(), (depth, o)


@needs_ref
def test_backbone_vs_reference_live():
    model = refload.load_model()
    data = small_batch([3000, 2000], seed=77)
    net = model.PointTransformerV3(in_channels=6, enable_flash=False, **SMALL_CFG).eval()
    sd = weights.fill_state_dict(net, prefix="ptv3.")
    with torch.inference_mode():
        torch.manual_seed(3)
        ref = net(dict(data)).feat
        torch.manual_seed(3)
        got = O.ptv3_forward(sd, data, SMALL_CFG)
    assert (ref - got).abs().max() < 1e-5


def _voxelize_inputs():
    """The seeded input generator stored beside the fixture (tests/golden/make_golden.py)."""
    src = open(os.path.join(GOLDEN, "make_golden.py")).read()
    ns = {}
    exec("import numpy as np\n" + src[src.index("def voxelize_inputs():"):src.index("def gen_voxelize(model):")], ns)
    return ns["voxelize_inputs"]()


def test_grid_coord_golden():
    """grid_coord derivation (model.py:94-96) against the reference's own Point."""
    coord, offset, grid_size = _voxelize_inputs()
    got = O.grid_coord_from_coord(torch.from_numpy(coord), grid_size)
    assert np.array_equal(got.numpy(), load("voxelize.npz")["grid_coord"])


def test_voxel_dedup_definition():
    """The oracle's dedup keeps exactly one point per (scene, voxel), the first one, in order."""
    g = torch.tensor([[0, 0, 0], [1, 0, 0], [0, 0, 0], [1, 0, 0], [0, 0, 0], [2, 2, 2]], dtype=torch.int32)
    b = torch.tensor([0, 0, 0, 1, 1, 1])
    keep, p2v, off = O.voxel_dedup(b, g, torch.tensor([3, 6]))
    assert keep.tolist() == [0, 1, 3, 4, 5]
    assert p2v.tolist() == [0, 1, 0, 2, 3, 4]
    assert off.tolist() == [2, 5]
