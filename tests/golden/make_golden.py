"""Generates the golden vectors under tests/golden from the UNMODIFIED reference
(serialization package imported directly; model.py imported through the
stand-in packages of oracle/refshim).  Run where the reference tree exists:

    python tests/golden/make_golden.py [serialization attention pooling backbone voxelize]

Inputs come from seeded generators (tests/helpers.py) and parameters from the
name-keyed fill of oracle/weights.py, so only outputs are stored."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import small_batch  # noqa: E402
from oracle import refload, weights  # noqa: E402

SMALL_CFG = dict(enc_depths=(1, 1, 1, 2, 1), enc_channels=(32, 32, 64, 64, 128), enc_num_head=(2, 2, 4, 4, 8),
                 enc_patch_size=(128,) * 5, dec_depths=(1, 1, 1, 1), dec_channels=(32, 32, 64, 64),
                 dec_num_head=(2, 2, 4, 4), dec_patch_size=(128,) * 4)
ORDERS = ["z", "z-trans", "hilbert", "hilbert-trans"]


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy()


def gen_serialization(ser, model):
    out = {}
    rng = np.random.default_rng(7)
    for depth in (1, 3, 9, 11, 16):
        g = rng.integers(-2, (1 << depth) + 2, size=(1500, 3)).astype(np.int32)
        b = rng.integers(0, 6, size=1500).astype(np.int64)
        out[f"grid_d{depth}"] = g
        out[f"batch_d{depth}"] = b
        for o in ORDERS:
            out[f"code_d{depth}_{o}"] = ser.encode(torch.from_numpy(g), torch.from_numpy(b), depth, o).numpy()
    # Point.serialization on de-duplicated voxels (no ties => argsort is well defined)
    data = small_batch([3000, 1700], seed=11)
    torch.manual_seed(5)
    pt = model.Point(dict(data))
    pt.serialization(order=ORDERS, shuffle_orders=True)
    out["point_code"] = pt.serialized_code.numpy()
    out["point_order"] = pt.serialized_order.numpy()
    out["point_inverse"] = pt.serialized_inverse.numpy()
    out["point_depth"] = np.int64(pt.serialized_depth)
    np.savez_compressed(os.path.join(HERE, "serialization.npz"), **out)


def gen_attention(model):
    out = {}
    for name, sizes, C, H, K in (("a", [1800], 32, 2, 128), ("b", [700, 90, 400], 64, 4, 256)):
        data = small_batch(sizes, seed=21)
        pt = model.Point(dict(data))
        pt.serialization(order=["hilbert", "z"], shuffle_orders=False)
        n = pt.batch.shape[0]
        feat = weights.keyed_tensor("attention.feat." + name, (n, C))
        att = model.SerializedAttention(C, H, K, order_index=1 if name == "b" else 0, enable_flash=False,
                                        upcast_attention=False, upcast_softmax=False).eval()
        weights.fill_state_dict(att, prefix="attention.%s." % name)
        with torch.inference_mode():
            pt.feat = feat
            out[name + "_fp32"] = att(pt).feat.numpy()
            pad, unpad, cu = att.get_padding_and_inverse(pt)
            out[name + "_pad"], out[name + "_unpad"], out[name + "_cu"] = pad.numpy(), unpad.numpy(), cu.numpy()
            att = att.bfloat16()
            pt.feat = feat.bfloat16()
            out[name + "_bf16"] = bf16_bits(att(pt).feat)
    # relative position bias (non-flash only), model.py:297-316, 468-469
    data = small_batch([900, 500], seed=23)
    pt = model.Point(dict(data))
    pt.serialization(order=["z"], shuffle_orders=False)
    att = model.SerializedAttention(32, 2, 128, enable_rpe=True, enable_flash=False, upcast_attention=False,
                                    upcast_softmax=False).eval()
    weights.fill_state_dict(att, prefix="attention.rpe.")
    with torch.inference_mode():
        pt.feat = weights.keyed_tensor("attention.feat.rpe", (pt.batch.shape[0], 32))
        out["rpe_fp32"] = att(pt).feat.numpy()
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **out)


def gen_pooling(model):
    out = {}
    data = small_batch([2500, 1200], seed=31)
    torch.manual_seed(9)
    pt = model.Point(dict(data))
    pt.serialization(order=ORDERS, shuffle_orders=True)
    n = pt.batch.shape[0]
    pt.feat = weights.keyed_tensor("pooling.feat", (n, 32))
    pt.sparsify()
    bn = lambda c: torch.nn.BatchNorm1d(c, eps=1e-3, momentum=0.01)
    pool = model.SerializedPooling(32, 64, stride=2, norm_layer=bn, act_layer=torch.nn.GELU).eval()
    up = model.SerializedUnpooling(64, 32, 48, norm_layer=bn, act_layer=torch.nn.GELU).eval()
    weights.fill_state_dict(pool, prefix="pooling.down.")
    weights.fill_state_dict(up, prefix="pooling.up.")
    with torch.inference_mode():
        c = pool(pt)
        for k in ("feat", "coord", "grid_coord", "batch", "serialized_code", "serialized_order",
                  "serialized_inverse", "pooling_inverse", "offset"):
            out["down_" + k] = c[k].numpy()
        out["down_depth"] = np.int64(c.serialized_depth)
        p = up(c)
        out["up_feat"] = p.feat.numpy()
        out["up_sparse_feat"] = p.sparse_conv_feat.features.numpy()
    np.savez_compressed(os.path.join(HERE, "pooling.npz"), **out)


def gen_backbone(model):
    out = {}
    data = small_batch([6000, 4000], seed=41)
    net = model.PointTransformerV3(in_channels=6, enable_flash=False, **SMALL_CFG).eval()
    weights.fill_state_dict(net, prefix="ptv3.")
    stage = {}

    def hook(name):
        def f(mod, inp, o):
            stage[name] = o.feat.detach().clone()
        return f
    for name in ("embedding", "enc.enc0", "enc.enc2", "enc.enc4", "dec.dec3", "dec.dec1"):
        net.get_submodule(name).register_forward_hook(hook(name))
    with torch.inference_mode():
        torch.manual_seed(1)
        o = net(dict(data))
        out["fp32"] = o.feat.numpy()
        for k, v in stage.items():
            out["fp32_" + k] = v.numpy()[:: max(1, v.shape[0] // 256)]   # row subsample
        out["order"] = o.serialized_order.numpy()
        net = net.bfloat16()
        d = dict(data)
        d["feat"] = d["feat"].bfloat16()
        torch.manual_seed(1)
        out["bf16"] = bf16_bits(net(d).feat)
    # per-dataset normalisation with context modulation (model.py:255-294), small cloud
    data = small_batch([1500, 1000], seed=43)
    net = model.PointTransformerV3(in_channels=6, enable_flash=False, pdnorm_bn=True, pdnorm_ln=True,
                                   pdnorm_adaptive=True, **SMALL_CFG).eval()
    weights.fill_state_dict(net, prefix="ptv3pd.")
    with torch.inference_mode():
        torch.manual_seed(2)
        d = dict(data, condition="S3DIS", context=weights.keyed_tensor("ptv3pd.context", (1, 256)))
        out["pdnorm_fp32"] = net(d).feat.numpy()
    np.savez_compressed(os.path.join(HERE, "backbone.npz"), **out)


def voxelize_inputs():
    """Seeded coordinates of two scenes (some negative, some sharing a voxel)."""
    rng = np.random.default_rng(51)
    coord = (rng.random((4000, 3)) * np.array([6.0, 5.0, 2.5]) - np.array([1.5, 0.0, 0.7])).astype(np.float32)
    coord[100:200] = coord[0:100] + np.float32(1e-4)           # near-duplicates: same voxel mostly
    offset = np.array([2600, 4000], dtype=np.int64)
    return coord, offset, 0.05


def gen_voxelize(model):
    # grid coordinates as Point derives them when only `coord` and `grid_size` are given (model.py:88-96)
    coord, offset, grid_size = voxelize_inputs()
    pt = model.Point({"coord": torch.from_numpy(coord), "offset": torch.from_numpy(offset),
                      "grid_size": grid_size, "feat": torch.zeros(coord.shape[0], 1)})
    pt.serialization(order=["z"])
    np.savez_compressed(os.path.join(HERE, "voxelize.npz"), grid_coord=pt.grid_coord.numpy().astype(np.int32))


def main():
    ser = refload.load_serialization()
    model = refload.load_model()
    assert ser is not None and model is not None, "the reference tree is required"
    only = set(sys.argv[1:])
    if not only or "serialization" in only:
        gen_serialization(ser, model)
    if not only or "attention" in only:
        gen_attention(model)
    if not only or "pooling" in only:
        gen_pooling(model)
    if not only or "backbone" in only:
        gen_backbone(model)
    if not only or "voxelize" in only:
        gen_voxelize(model)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    main()
