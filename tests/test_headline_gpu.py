"""Parity of the CUDA path with the CPU oracle at the sizes the benchmark runs:
the default backbone in bf16 on the four-scene indoor batch (wide levels of 256
and 512 channels, 32 heads, patch 1024, ``enable_flash=True``), the xCPE operator
chain at 80 000 voxels and 128 channels, and one shard of the LiDAR-like batch.

Index work (serialized codes and orders of every level, pooling clusters, kernel
maps) must be bit-exact.  Features are compared stage by stage: the oracle is run
in bf16 and in fp32, the distance between those two runs is the noise floor of
bf16 itself at that depth of the network, and the CUDA path has to stay within a
small factor of it (the same rule the small-configuration tests use)."""
import pytest
import torch
import torch.nn.functional as F

from helpers import TOL, assert_close, assert_close_chain, rel_l2
from oracle import ptv3_oracle as O
import pointtransformerv3_b200 as P
from pointtransformerv3_b200 import ops, synthetic

pytestmark = pytest.mark.gpu

STAGES = ("embedding", "enc.enc0", "enc.enc1", "enc.enc2", "enc.enc3", "enc.enc4",
          "dec.dec3", "dec.dec2", "dec.dec1", "dec.dec0")


def _run_cuda(net, data, dtype):
    """Forward on the GPU with a hook on the last module of every stage (the backbone calls the
    modules of its first stage one by one, so the stage container itself is not always called);
    returns (output Point, {stage: (snapshot of the Point's entries, its features)}): later modules
    mutate the Point objects (the unpooling pops the pooling entries)."""
    seen = {}
    hooks = []
    for name in STAGES:
        stage = net.get_submodule(name)
        last = stage if name == "embedding" else list(stage._modules.values())[-1]
        hooks.append(last.register_forward_hook(
            lambda m, i, o, name=name: seen.__setitem__(name, (P.point.AttrDict(o), o.feat.detach().clone()))))
    d = {k: v.cuda() for k, v in data.items()}
    d["feat"] = d["feat"].to(dtype)
    with torch.inference_mode():
        torch.manual_seed(1)
        out = net(d)
    for h in hooks:
        h.remove()
    return out, seen


def _check_backbone(data, in_channels, flash=True):
    torch.manual_seed(0)
    net = P.PointTransformerV3(in_channels=in_channels, enable_flash=flash).eval()
    sd32 = {k: v.clone() for k, v in net.state_dict().items()}
    sd16 = {k: (v.bfloat16() if v.is_floating_point() else v) for k, v in sd32.items()}
    net = net.cuda().bfloat16()
    out, seen = _run_cuda(net, data, torch.bfloat16)

    torch.set_num_threads(max(1, torch.get_num_threads()))
    taps16, taps32 = {}, {}
    d16 = dict(data, feat=data["feat"].bfloat16())
    with torch.inference_mode():
        torch.manual_seed(1)
        ref16, levels = O.ptv3_forward(sd16, d16, dict(in_channels=in_channels), return_levels=True,
                                       flash=flash, taps=taps16)
        torch.manual_seed(1)
        ref32 = O.ptv3_forward(sd32, data, dict(in_channels=in_channels), flash=flash, taps=taps32)

    # ---- index work: bit-exact at every level ---------------------------------------
    for s, lv in enumerate(levels):
        pt = seen["enc.enc%d" % s][0]
        assert pt.serialized_depth == lv.depth
        assert torch.equal(pt.serialized_code.cpu(), lv.code), "codes of level %d" % s
        assert torch.equal(pt.serialized_order.cpu(), lv.order), "orders of level %d" % s
        assert torch.equal(pt.serialized_inverse.cpu(), lv.inverse), "inverses of level %d" % s
        assert torch.equal(pt.grid_coord.cpu().long(), lv.grid_coord.long()), "grid of level %d" % s
        assert torch.equal(pt.batch.cpu(), lv.batch), "scene ids of level %d" % s
        if s > 0:
            assert torch.equal(pt.pooling_inverse.cpu(), lv.cluster), "clusters of level %d" % s
        nbr = ops.kmap_build(pt.sparse_conv_feat.indices, 3)
        assert torch.equal(nbr.t().cpu().long(), lv.nbr3), "kernel map of level %d" % s

    # ---- features, stage by stage ------------------------------------------------------
    report = {}
    for name in STAGES:
        got = seen[name][1].float().cpu()
        r16, r32 = taps16[name].float(), taps32[name].float()
        assert got.shape == r32.shape, name
        floor = rel_l2(r16, r32)
        err32, err16 = rel_l2(got, r32), rel_l2(got, r16)
        report[name] = (floor, err32, err16)
        assert err32 <= 1.5 * floor + 2e-3, "%s: %.3g from the fp32 oracle, bf16 oracle itself %.3g" % (
            name, err32, floor)
        assert err16 <= 2.0 * floor + 2e-3, "%s: %.3g from the bf16 oracle (floor %.3g)" % (name, err16, floor)
    floor = rel_l2(ref16, ref32)
    assert rel_l2(out.feat, ref32) <= 1.5 * floor + 2e-3
    assert bool(torch.isfinite(out.feat.float()).all())
    return report


def test_default_backbone_bf16_on_the_bench_batch():
    """BASELINE configuration 4: the workload `bench.py` times."""
    data = synthetic.indoor_batch(4, first_seed=0, target_voxels=100_000, grid_size=0.02)
    assert 380_000 < int(data["offset"][-1]) < 440_000
    _check_backbone(data, 6, flash=True)


def test_default_backbone_bf16_on_a_lidar_shard():
    """BASELINE configuration 5, one GPU's share at 8 GPUs: two LiDAR-like scenes,
    grid 0.05, four input channels."""
    data = synthetic.lidar_batch(2, first_seed=0, grid_size=0.05)
    assert data["feat"].shape[1] == 4
    _check_backbone(data, 4, flash=True)


def test_xcpe_chain_at_config3_size():
    """BASELINE configuration 3 at its size: kernel map, 3x3x3 submanifold convolution with
    128 channels on ~80 000 voxels, then Linear + LayerNorm + residual, in bf16."""
    C = 128
    coord, gc = synthetic.indoor_scene(0, 80_000, 0.02)
    n = gc.shape[0]
    assert 70_000 < n < 95_000
    g = torch.Generator().manual_seed(0)
    feat = torch.randn(n, C, generator=g)
    w = torch.randn(C, 3, 3, 3, C, generator=g) / (9 * C) ** 0.5
    b = torch.randn(C, generator=g) * 0.1
    wl = torch.randn(C, C, generator=g) / C ** 0.5
    bl = torch.randn(C, generator=g) * 0.1
    lw, lb = 1 + 0.1 * torch.randn(C, generator=g), 0.1 * torch.randn(C, generator=g)
    ind = torch.cat([torch.zeros(n, 1, dtype=torch.int32), gc], 1).contiguous()

    nbr_ref = O.kernel_map(ind, 3)

    def chain(cast):
        x = O.subm_conv(cast(feat), nbr_ref, cast(w), cast(b))
        x = F.linear(x, cast(wl), cast(bl))
        return cast(feat) + F.layer_norm(x, (C,), cast(lw), cast(lb), 1e-5), x
    ref32, _ = chain(lambda t: t.float())
    ref16, _ = chain(lambda t: t.bfloat16())

    dev = lambda t: t.bfloat16().cuda()
    nbr = ops.kmap_build(ind.cuda(), 3)
    assert torch.equal(nbr.t().cpu().long(), nbr_ref), "kernel map"
    codes = ops.encode(gc.cuda(), torch.zeros(n, dtype=torch.int64, device="cuda"), 9, ["z"])
    order, _ = ops.argsort_inverse(codes, 28)
    conv = ops.subm_conv(dev(feat), nbr.index_select(1, order[0]), dev(w), dev(b), row_order=order[0])
    ref_conv = O.subm_conv(feat.bfloat16(), nbr_ref, w.bfloat16(), b.bfloat16())
    assert_close(conv, ref_conv, what="convolution", **TOL[torch.bfloat16])
    ln = torch.nn.LayerNorm(C)
    ln.weight.data, ln.bias.data = lw.clone(), lb.clone()
    ln = ln.cuda().bfloat16()
    ident = torch.nn.LayerNorm(C).cuda().bfloat16()      # second norm of the fused kernel, unused here
    got, _ = ops.linear_ln(conv, dev(wl), dev(bl), dev(feat), ln, ident)
    floor = rel_l2(ref16, ref32)
    assert rel_l2(got, ref32) <= 1.5 * floor + 1e-3
    # three operators and a residual sum: all but 1e-6 of the elements within the one-operator
    # tolerance (measured: 1 of 10.8 M outside, by one bf16 ulp of an operand of a cancelling sum)
    assert_close_chain(got, ref16, what="convolution + Linear + LayerNorm + residual", frac=1e-6,
                       **TOL[torch.bfloat16])
