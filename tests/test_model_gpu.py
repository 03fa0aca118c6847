"""Module- and backbone-level parity of the CUDA-backed modules with the golden
vectors of the reference and with the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from helpers import TOL, assert_close, assert_close_chain, rel_l2, small_batch
from oracle import ptv3_oracle as O, weights
import pointtransformerv3_b200 as P

pytestmark = pytest.mark.gpu
ORDERS = ["z", "z-trans", "hilbert", "hilbert-trans"]
SMALL_CFG = dict(enc_depths=(1, 1, 1, 2, 1), enc_channels=(32, 32, 64, 64, 128), enc_num_head=(2, 2, 4, 4, 8),
                 enc_patch_size=(128,) * 5, dec_depths=(1, 1, 1, 1), dec_channels=(32, 32, 64, 64),
                 dec_num_head=(2, 2, 4, 4), dec_patch_size=(128,) * 4)


def load(name):
    return np.load(os.path.join(GOLDEN, name))


def from_bf16_bits(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def cuda_data(data, dtype=None):
    d = {k: v.cuda() for k, v in data.items()}
    if dtype is not None:
        d["feat"] = d["feat"].to(dtype)
    return d


def test_point_serialization_golden():
    g = load("serialization.npz")
    data = small_batch([3000, 1700], seed=11)
    torch.manual_seed(5)
    pt = P.Point(cuda_data(data))
    pt.serialization(order=ORDERS, shuffle_orders=True)
    assert pt.serialized_depth == int(g["point_depth"])
    assert (pt.serialized_code.cpu().numpy() == g["point_code"]).all()
    assert (pt.serialized_order.cpu().numpy() == g["point_order"]).all()
    assert (pt.serialized_inverse.cpu().numpy() == g["point_inverse"]).all()


def test_serialization_api_golden():
    g = load("serialization.npz")
    for depth in (1, 3, 9, 11, 16):
        grid = torch.from_numpy(g[f"grid_d{depth}"]).cuda()
        batch = torch.from_numpy(g[f"batch_d{depth}"]).cuda()
        for o in ORDERS:
            got = P.serialization.encode(grid, batch, depth, o)
            assert (got.cpu().numpy() == g[f"code_d{depth}_{o}"]).all(), (depth, o)


@pytest.mark.parametrize("name,sizes,C,H,K,oi", [("a", [1800], 32, 2, 128, 0), ("b", [700, 90, 400], 64, 4, 256, 1)])
def test_attention_module_golden(name, sizes, C, H, K, oi):
    g = load("attention.npz")
    data = small_batch(sizes, seed=21)
    pt = P.Point(cuda_data(data))
    pt.serialization(order=["hilbert", "z"], shuffle_orders=False)
    n = pt.batch.shape[0]
    feat = weights.keyed_tensor("attention.feat." + name, (n, C))
    att = P.SerializedAttention(C, H, K, order_index=oi, enable_flash=False, upcast_attention=False,
                                upcast_softmax=False).eval()
    weights.fill_state_dict(att, prefix="attention.%s." % name)
    att = att.cuda()
    with torch.inference_mode():
        pt.feat = feat.cuda()
        out = att(pt).feat
        pad, unpad, cu = att.get_padding_and_inverse(pt)
        assert (pad.cpu().numpy() == g[name + "_pad"]).all()
        assert (unpad.cpu().numpy() == g[name + "_unpad"]).all()
        assert (cu.cpu().numpy() == g[name + "_cu"]).all()
        ref = torch.from_numpy(g[name + "_fp32"])
        assert_close(out, ref, what="attention fp32", **TOL[torch.float32])
        att = att.bfloat16()
        pt.feat = feat.cuda().bfloat16()
        out16 = att(pt).feat
        assert_close(out16, from_bf16_bits(g[name + "_bf16"]), what="attention bf16", **TOL[torch.bfloat16])
        assert rel_l2(out16, ref) < 1e-2


def test_pooling_modules_golden():
    g = load("pooling.npz")
    data = small_batch([2500, 1200], seed=31)
    torch.manual_seed(9)
    pt = P.Point(cuda_data(data))
    pt.serialization(order=ORDERS, shuffle_orders=True)
    n = pt.batch.shape[0]
    pt.feat = weights.keyed_tensor("pooling.feat", (n, 32)).cuda()
    pt.sparsify()
    bn = lambda c: torch.nn.BatchNorm1d(c, eps=1e-3, momentum=0.01)
    pool = P.GridPooling(32, 64, stride=2, norm_layer=bn, act_layer=torch.nn.GELU).eval()
    up = P.GridUnpooling(64, 32, 48, norm_layer=bn, act_layer=torch.nn.GELU).eval()
    weights.fill_state_dict(pool, prefix="pooling.down.")
    weights.fill_state_dict(up, prefix="pooling.up.")
    pool, up = pool.cuda(), up.cuda()
    with torch.inference_mode():
        c = pool(pt)
        for k in ("grid_coord", "batch", "serialized_code", "serialized_order", "serialized_inverse",
                  "pooling_inverse", "offset"):
            assert (c[k].cpu().numpy() == g["down_" + k]).all(), k
        assert c.serialized_depth == int(g["down_depth"])
        assert_close(c.feat, torch.from_numpy(g["down_feat"]), what="pooled feat", **TOL[torch.float32])
        assert_close(c.coord, torch.from_numpy(g["down_coord"]), atol=1e-5, rtol=1e-5, what="pooled coord")
        p = up(c)
        assert_close(p.feat, torch.from_numpy(g["up_feat"]), what="unpooled feat", **TOL[torch.float32])
        assert_close(p.sparse_conv_feat.features, torch.from_numpy(g["up_sparse_feat"]),
                     what="sparse tensor after unpooling", **TOL[torch.float32])


def _small_net(dtype):
    net = P.PointTransformerV3(in_channels=6, enable_flash=False, **SMALL_CFG).eval()
    sd = weights.fill_state_dict(net, prefix="ptv3.")
    return net.cuda().to(dtype), sd


def test_backbone_golden_fp32():
    g = load("backbone.npz")
    data = small_batch([6000, 4000], seed=41)
    net, _ = _small_net(torch.float32)
    stage = {}
    for name in ("embedding", "enc.enc0", "enc.enc2", "enc.enc4", "dec.dec3", "dec.dec1"):
        net.get_submodule(name).register_forward_hook(
            lambda m, i, o, name=name: stage.__setitem__(name, o.feat.detach().clone()))
    with torch.inference_mode():
        torch.manual_seed(1)
        out = net(cuda_data(data))
    assert (out.serialized_order.cpu().numpy() == g["order"]).all()
    for k, v in stage.items():
        ref = torch.from_numpy(g["fp32_" + k])
        assert_close(v[:: max(1, v.shape[0] // 256)], ref, atol=2e-4, rtol=2e-4, what=k)
    # 11 blocks deep: errors of the order of 1e-6 per operator accumulate
    assert_close(out.feat, torch.from_numpy(g["fp32"]), atol=5e-4, rtol=5e-4, what="backbone fp32")
    assert rel_l2(out.feat, torch.from_numpy(g["fp32"])) < 1e-5


def test_backbone_golden_bf16():
    """End to end in bf16 the reference differs from its own fp32 run by far more
    than the per-operator tolerance, so the bound here is relative to that noise
    floor: the CUDA path must be as close to the fp32 reference as the bf16
    reference is (up to a factor), and close to the bf16 reference itself."""
    g = load("backbone.npz")
    data = small_batch([6000, 4000], seed=41)
    net, _ = _small_net(torch.bfloat16)
    with torch.inference_mode():
        torch.manual_seed(1)
        out = net(cuda_data(data, torch.bfloat16)).feat
    ref32 = torch.from_numpy(g["fp32"])
    ref16 = from_bf16_bits(g["bf16"]).float()
    floor = rel_l2(ref16, ref32)
    assert rel_l2(out, ref32) <= 1.5 * floor + 1e-3, (rel_l2(out, ref32), floor)
    assert rel_l2(out, ref16) <= 2.0 * floor + 1e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_vs_oracle(dtype):
    """One Block (xCPE + attention + MLP) on identical inputs against the oracle."""
    data = small_batch([5000, 2000], seed=51)
    C, H, K = 64, 4, 1024
    blk = P.Block(C, H, K, order_index=2, cpe_indice_key="s", enable_flash=False, upcast_attention=False,
                  upcast_softmax=False).eval()
    sd = weights.fill_state_dict(blk, prefix="blk.")
    sd = {("b." + k): v.to(dtype) for k, v in sd.items()}
    pt = P.Point(cuda_data(data))
    pt.serialization(order=ORDERS, shuffle_orders=False)
    n = pt.batch.shape[0]
    feat = weights.keyed_tensor("blk.feat", (n, C)).to(dtype)
    pt.feat = feat.cuda()
    pt.sparsify()
    with torch.inference_mode():
        got = blk.cuda().to(dtype)(pt).feat
    batch = O.offset_to_batch(data["offset"])
    code, order, inverse, depth = O.serialization(data["grid_coord"], batch, ORDERS)
    lv = O.Level(coord=data["coord"], grid_coord=data["grid_coord"], batch=batch, offset=data["offset"],
                 code=code, order=order, inverse=inverse, depth=depth, cluster=None, parent=None)
    ref = O.block(sd, "b.", lv, feat, H, K, 2)
    if dtype == torch.float32:
        assert_close(got, ref, atol=2e-4, rtol=2e-4, what="block fp32")
    else:
        ref32 = O.block({k: v.float() for k, v in sd.items()}, "b.", lv, feat.float(), H, K, 2)
        assert rel_l2(got, ref32) <= 1.5 * rel_l2(ref, ref32) + 1e-3
        # nine bf16 operators in a chain: see assert_close_chain
        assert_close_chain(got, ref, what="block bf16", **TOL[torch.bfloat16])


def test_flash_flag_uses_full_patch_and_short_sequences():
    """enable_flash=True keeps patch = patch_size; scenes shorter than the patch
    become one short sequence (model.py:394-404, :476-483)."""
    data = small_batch([900, 300], seed=61)
    C, H, K = 32, 2, 256
    att = P.SerializedAttention(C, H, K, enable_flash=True, upcast_attention=False, upcast_softmax=False).eval()
    sd = weights.fill_state_dict(att, prefix="fl.")
    pt = P.Point(cuda_data(data))
    pt.serialization(order=["z"], shuffle_orders=False)
    n = pt.batch.shape[0]
    feat = weights.keyed_tensor("fl.feat", (n, C))
    pt.feat = feat.cuda()
    with torch.inference_mode():
        got = att.cuda()(pt).feat.cpu()
    # oracle: varlen attention written directly from the padded layout
    counts = O.offset_to_counts(data["offset"]).tolist()
    pad, unpad, cu = O.pad_plan(data["offset"], K)
    order, inverse = pt.serialized_order[0].cpu(), pt.serialized_inverse[0].cpu()
    qkv = torch.nn.functional.linear(feat, sd["qkv.weight"], sd["qkv.bias"])[order[pad]]
    outp = torch.empty(qkv.shape[0], C)
    for s in range(len(cu) - 1):
        a, b = int(cu[s]), int(cu[s + 1])
        q, k, v = qkv[a:b].reshape(b - a, 3, H, C // H).permute(1, 2, 0, 3)
        w = torch.softmax((q * (C // H) ** -0.5) @ k.transpose(-1, -2), -1)
        outp[a:b] = (w @ v).transpose(0, 1).reshape(b - a, C)
    ref = torch.nn.functional.linear(outp[unpad[inverse]], sd["proj.weight"], sd["proj.bias"])
    assert_close(got, ref, what="varlen attention", **TOL[torch.float32])


def test_lidar_like_scenes_vs_oracle():
    """Sparse outdoor-like sweeps (grid 0.05, 4 input channels, three scenes): the
    whole small backbone against the CPU oracle in fp32."""
    from pointtransformerv3_b200 import synthetic
    scenes = [synthetic.lidar_scene(seed=s, grid_size=0.05, n_sweeps=1, beams=32, azimuth_steps=256)
              for s in (0, 1, 2)]
    data = synthetic.make_batch(scenes, 1, 0)
    cfg = dict(SMALL_CFG, enc_patch_size=(256,) * 5, dec_patch_size=(256,) * 4)
    net = P.PointTransformerV3(in_channels=4, enable_flash=False, **cfg).eval()
    sd = weights.fill_state_dict(net, prefix="lidar.")
    net = net.cuda()
    with torch.inference_mode():
        torch.manual_seed(3)
        out = net(cuda_data(data))
        torch.manual_seed(3)
        ref, levels = O.ptv3_forward(sd, data, dict(cfg, in_channels=4), return_levels=True)
    assert torch.equal(out.serialized_order.cpu(), levels[0].order)
    assert torch.equal(out.serialized_code.cpu(), levels[0].code)
    assert_close(out.feat, ref, atol=5e-4, rtol=5e-4, what="lidar-like backbone fp32")


@pytest.mark.parametrize("flash", [False, True])
def test_encoder_and_decoder_patch_sizes_differ(flash):
    """Encoder patch 256, decoder patch 128: the blocks of one level then need two padding
    plans.  The reference would reuse the cached one (model.py:387-391); here the plan is
    rebuilt for the block's own patch size, which is what the oracle (a fresh plan per
    block) computes."""
    data = small_batch([3000, 1400], seed=81)
    cfg = dict(SMALL_CFG, enc_patch_size=(256,) * 5, dec_patch_size=(128,) * 4)
    net = P.PointTransformerV3(in_channels=6, enable_flash=flash, **cfg).eval()
    sd = weights.fill_state_dict(net, prefix="patchmix.")
    net = net.cuda()
    with torch.inference_mode():
        torch.manual_seed(4)
        out = net(cuda_data(data))
        torch.manual_seed(4)
        ref = O.ptv3_forward(sd, data, cfg, flash=flash)
    assert_close(out.feat, ref, atol=5e-4, rtol=5e-4, what="mixed patch sizes, fp32")
    net = net.bfloat16()
    with torch.inference_mode():
        torch.manual_seed(4)
        out16 = net(cuda_data(data, torch.bfloat16))
    assert rel_l2(out16.feat, ref) < 3e-2


def test_cls_mode_and_single_order():
    """Encoder-only mode with one serialization order and no shuffling."""
    data = small_batch([3000, 1500], seed=71)
    cfg = dict(enc_depths=(1, 1, 1, 1, 1), enc_channels=(32, 32, 64, 64, 128), enc_num_head=(2, 2, 4, 4, 8),
               enc_patch_size=(128,) * 5, cls_mode=True, order="hilbert", shuffle_orders=False)
    net = P.PointTransformerV3(in_channels=6, enable_flash=False, **cfg).eval()
    sd = weights.fill_state_dict(net, prefix="cls.")
    net = net.cuda()
    with torch.inference_mode():
        out = net(cuda_data(data))
        ocfg = dict(cfg, order=("hilbert",), dec_depths=(), dec_channels=(), dec_num_head=(), dec_patch_size=())
        ref = O.ptv3_forward(sd, data, ocfg)
    assert out.feat.shape == ref.shape
    assert_close(out.feat, ref, atol=5e-4, rtol=5e-4, what="encoder-only backbone")


@pytest.mark.parametrize("sizes", [[1, 60, 2500], [7], [300, 300]])
def test_tiny_and_ragged_scenes_vs_oracle(sizes):
    """Scenes of one point, scenes smaller than a patch, a single tiny scene: the
    non-flash rule K = min(smallest scene, patch) degenerates gracefully
    (model.py:441-444) and pooling levels shrink to a handful of voxels."""
    data = small_batch(sizes, seed=sum(sizes))
    cfg = dict(SMALL_CFG)
    net = P.PointTransformerV3(in_channels=6, enable_flash=False, **cfg).eval()
    sd = weights.fill_state_dict(net, prefix="tiny.")
    net = net.cuda()
    with torch.inference_mode():
        torch.manual_seed(11)
        out = net(cuda_data(data))
        torch.manual_seed(11)
        ref = O.ptv3_forward(sd, data, cfg)
    assert out.feat.shape == ref.shape
    assert_close(out.feat, ref, atol=5e-4, rtol=5e-4, what="tiny scenes")


def test_empty_inputs_are_accepted_by_the_operators():
    """n = 0 through the C ABI: every operator returns without launching."""
    dev = torch.device("cuda")
    e = lambda *shape, dtype=torch.float32: torch.empty(*shape, dtype=dtype, device=dev)
    from pointtransformerv3_b200 import ops
    assert ops.encode(e(0, 3, dtype=torch.int32), None, 16, ["z", "hilbert"]).shape == (2, 0)
    order, inverse = ops.argsort_inverse(e(4, 0, dtype=torch.int64), 30)
    assert order.shape == (4, 0) and inverse.shape == (4, 0)
    assert ops.kmap_build(e(0, 4, dtype=torch.int32), 3).shape == (27, 0)
    assert ops.subm_conv(e(0, 32), e(27, 0, dtype=torch.int32), e(32, 3, 3, 3, 32), e(32)).shape == (0, 32)
    s, y = ops.add_layernorm(e(0, 32), e(0, 32), None, torch.nn.LayerNorm(32).cuda())
    assert s.shape == (0, 32) and y.shape == (0, 32)
    grid, batch = ops.decode(e(0, dtype=torch.int64), 9, "hilbert")
    assert grid.shape == (0, 3) and batch.shape == (0,)


def test_bad_arguments_raise_with_a_message():
    """Host-side failure injection: wrong shapes / dtypes / sizes come back as a
    Ptv3Error (or ValueError) carrying the library's message, never as a crash."""
    from pointtransformerv3_b200 import _lib, ops
    g = torch.zeros(10, 3, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.Ptv3Error, match="depth"):
        ops.encode(g, None, 17, ["z"])
    with pytest.raises(ValueError):
        ops.encode(torch.zeros(10, 2, dtype=torch.int32, device="cuda"), None, 8, ["z"])
    with pytest.raises(_lib.Ptv3Error, match="head dim"):
        qkv = torch.zeros(10, 3 * 24, device="cuda")
        pad, unpad, cu = ops.pad_plan(torch.tensor([10], device="cuda"), [10], 10)
        ops.attention(qkv, torch.arange(10, device="cuda"), pad, unpad, cu, 2, 10, 1.0)
    with pytest.raises(_lib.Ptv3Error, match="status"):
        # the totals the caller states do not match the offsets: the kernel reports it
        ops.pad_plan(torch.tensor([10], device="cuda"), [12], 4)
    with pytest.raises(_lib.Ptv3Error, match="status"):
        ops.kmap_build(torch.tensor([[0, 70000, 0, 0]], dtype=torch.int32, device="cuda"), 3)
    with pytest.raises(_lib.Ptv3Error):
        ops.mlp(torch.zeros(8, 48, device="cuda").bfloat16(), torch.zeros(192, 48, device="cuda").bfloat16(),
                torch.zeros(192, device="cuda").bfloat16(), torch.zeros(48, 192, device="cuda").bfloat16(),
                torch.zeros(48, device="cuda").bfloat16(), torch.zeros(8, 48, device="cuda").bfloat16())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_relative_position_bias(dtype):
    """enable_rpe=True (non-flash): golden vector of the reference in fp32, oracle in bf16."""
    g = load("attention.npz")
    data = small_batch([900, 500], seed=23)
    pt = P.Point(cuda_data(data))
    pt.serialization(order=["z"], shuffle_orders=False)
    att = P.SerializedAttention(32, 2, 128, enable_rpe=True, enable_flash=False, upcast_attention=False,
                                upcast_softmax=False).eval()
    sd = weights.fill_state_dict(att, prefix="attention.rpe.")
    feat = weights.keyed_tensor("attention.feat.rpe", (pt.batch.shape[0], 32))
    att = att.cuda().to(dtype)
    with torch.inference_mode():
        pt.feat = feat.cuda().to(dtype)
        got = att(pt).feat
    if dtype == torch.float32:
        assert_close(got, torch.from_numpy(g["rpe_fp32"]), what="rpe attention fp32", **TOL[torch.float32])
    else:
        c = lambda k: sd[k].to(dtype)
        ref = O.attention(feat.to(dtype), c("qkv.weight"), c("qkv.bias"), c("proj.weight"), c("proj.bias"),
                          pt.serialized_order[0].cpu(), pt.serialized_inverse[0].cpu(), data["offset"], 2, 128,
                          rpe=(data["grid_coord"], c("rpe.rpe_table"), att.rpe.pos_bnd))
        assert_close(got, ref, what="rpe attention bf16", **TOL[torch.bfloat16])


def test_backbone_with_per_dataset_norm_golden():
    """pdnorm_bn / pdnorm_ln / pdnorm_adaptive (model.py:255-294, 834-857): the generic module
    path with the CUDA point operators, against the reference's output."""
    g = load("backbone.npz")
    data = small_batch([1500, 1000], seed=43)
    net = P.PointTransformerV3(in_channels=6, enable_flash=False, pdnorm_bn=True, pdnorm_ln=True,
                               pdnorm_adaptive=True, **SMALL_CFG).eval()
    weights.fill_state_dict(net, prefix="ptv3pd.")
    net = net.cuda()
    d = cuda_data(data)
    d["condition"] = "S3DIS"
    d["context"] = weights.keyed_tensor("ptv3pd.context", (1, 256)).cuda()
    with torch.inference_mode():
        torch.manual_seed(2)
        out = net(d).feat
    assert_close(out, torch.from_numpy(g["pdnorm_fp32"]), atol=5e-4, rtol=5e-4, what="PDNorm backbone")


@pytest.mark.gpu
@pytest.mark.parametrize("channels,heads,n_per_scene", [(32, 2, 3000), (64, 4, 2500), (128, 8, 1500),
                                                       (256, 16, 900), (512, 32, 400)])
def test_block_single_call_matches_per_operator_path(channels, heads, n_per_scene):
    """ptv3_block_fwd (one C call per block) against the same block run operator by
    operator from Python (the path per-operator timing takes): same kernels for
    C <= 128, cuBLASLt instead of torch's GEMM calls above."""
    from pointtransformerv3_b200 import ops
    from pointtransformerv3_b200.model import Block
    from pointtransformerv3_b200.point import Point
    data = small_batch([n_per_scene, n_per_scene // 2], 21)
    torch.manual_seed(channels)
    blk = Block(channels, heads, patch_size=1024, cpe_indice_key="t", order_index=0, upcast_attention=False,
                upcast_softmax=False).eval().cuda().bfloat16()
    feat = torch.randn(data["grid_coord"].shape[0], channels).bfloat16().cuda()

    def run(per_operator):
        p = Point({"feat": feat.clone(), "grid_coord": data["grid_coord"].cuda(), "offset": data["offset"].cuda()})
        p.serialization(order=["z", "hilbert"], shuffle_orders=False)
        p.sparsify()
        ops.TIMERS = {} if per_operator else None
        try:
            with torch.inference_mode():
                out = blk(p).feat
        finally:
            ops.TIMERS = None
        return out

    a, b = run(True), run(False)
    assert bool(torch.isfinite(b.float()).all())
    assert rel_l2(b, a) < 4e-3, rel_l2(b, a)


@pytest.mark.gpu
def test_forward_with_host_metadata_and_deferred_status():
    """The optional entries that let a caller skip the host waits of a pass (scene sizes,
    code depth and sparse shape known on the host; status word read later) do not change
    the result."""
    data = small_batch([3000, 1800], 33)
    torch.manual_seed(0)
    net = P.PointTransformerV3(in_channels=6, enc_depths=(1, 1, 1, 1, 1), dec_depths=(1, 1, 1, 1)).eval().cuda()
    dev = {k: v.cuda() for k, v in data.items()}
    with torch.inference_mode():
        torch.manual_seed(1)
        ref = net(dict(dev)).feat
        mx = data["grid_coord"].max(0).values.tolist()
        meta = {"offset_host": data["offset"].tolist(), "serialization_depth": max(mx).bit_length(),
                "sparse_shape": [v + 96 for v in mx]}
        net.defer_status_check = True
        torch.manual_seed(1)
        point = net(dict(dev, **meta))
        point.check_status("deferred", force=True)
        net.defer_status_check = False
    assert torch.equal(point.feat, ref)


@pytest.mark.gpu
def test_repeated_passes_over_changing_batches_are_bit_identical():
    """Batches of different shapes interleaved and repeated, on the default path: every kernel
    is deterministic (the convolutions sum a tile's offsets in tensor memory in a fixed order),
    so any difference between repeats would be a hazard between the planning stream, the feature
    stream and the allocator (plans are made two stages ahead on a second stream)."""
    torch.manual_seed(0)
    net = P.PointTransformerV3(in_channels=6).eval().cuda().bfloat16()
    batches = []
    for i, sizes in enumerate(([900], [4000, 2500, 700], [12000, 300], [150, 150, 150, 150, 9000])):
        d = small_batch(sizes, 50 + i)
        d["feat"] = d["feat"].bfloat16()
        batches.append({k: v.cuda() for k, v in d.items()})

    def run(d):
        with torch.inference_mode():
            torch.manual_seed(1)
            return net(dict(d)).feat

    first = [run(d).clone() for d in batches]
    for order in ([3, 0, 2, 1], [1, 1, 3, 0], [2, 3, 0, 2]):
        for i in order:
            assert torch.equal(run(batches[i]), first[i]), "batch %d differs between repeats" % i


def test_bench_batch_is_bit_identical_between_passes():
    """The benchmark's batch (coarse levels of 27 000, 7 000 and 2 000 voxels) gives the same bits on
    three passes."""
    from pointtransformerv3_b200 import synthetic
    data = synthetic.indoor_batch(4, first_seed=0, target_voxels=100_000, grid_size=0.02, dtype=torch.bfloat16)
    d = {k: v.cuda() for k, v in data.items()}
    torch.manual_seed(0)
    net = P.PointTransformerV3(in_channels=6).eval().cuda().bfloat16()
    outs = []
    for _ in range(3):
        with torch.inference_mode():
            torch.manual_seed(1)
            outs.append(net(dict(d)).feat.clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.gpu
def test_pair_list_convolution_in_the_backbone(monkeypatch):
    """The pair-list convolution (fixed-point atomic accumulation), which the default backbone does
    not reach at its widths, taken from 128 channels up: same result as the kernel-map convolution
    within the bf16 tolerance of a whole backbone, and the same bits on two passes."""
    from pointtransformerv3_b200 import sparse
    d = small_batch([5000, 2500, 1200], 77)
    d["feat"] = d["feat"].bfloat16()
    dev = {k: v.cuda() for k, v in d.items()}
    torch.manual_seed(0)
    net = P.PointTransformerV3(in_channels=6).eval().cuda().bfloat16()

    def run():
        with torch.inference_mode():
            torch.manual_seed(1)
            return net(dict(dev)).feat.clone()

    base = run()
    monkeypatch.setattr(sparse, "PAIR_PATH_MIN_CHANNELS", 128)
    got, again = run(), run()
    assert torch.equal(got, again)
    assert rel_l2(got, base) < 2e-2
