"""Torch-on-CPU restatement of the Point Transformer V3 inference path.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``): the checker the CUDA
path is compared with, and the timed CPU baseline.  It is written as plain
functions over a ``state_dict`` so that it shares no code with the shipped
modules.  Each function cites the reference lines it restates
(paths are relative to the reference project's root).
"""
import math

import numpy as np
import torch
import torch.nn.functional as F

from . import cenc

ORDERS = ("z", "z-trans", "hilbert", "hilbert-trans")


# --------------------------------------------------------------------------- #
# model.py:28-45  offset/batch helpers
# --------------------------------------------------------------------------- #
def offset_to_counts(offset):
    o = offset.to(torch.int64)
    return torch.diff(o, prepend=torch.zeros(1, dtype=torch.int64))


def offset_to_batch(offset):
    c = offset_to_counts(offset)
    return torch.repeat_interleave(torch.arange(len(c), dtype=torch.int64), c)


def batch_to_offset(batch):
    return torch.cumsum(torch.bincount(batch), 0).to(torch.int64)


# --------------------------------------------------------------------------- #
# model.py:81-136  Point.serialization
# --------------------------------------------------------------------------- #
def grid_coord_from_coord(coord, grid_size):
    """model.py:94-96 (and 156-158): grid_coord = trunc((coord - coord.min(0)) / grid_size).int(),
    the minimum taken over the whole batch."""
    coord = coord.to(torch.float32)
    return torch.div(coord - coord.min(0)[0], grid_size, rounding_mode="trunc").int()


def voxel_dedup(batch, grid_coord, offset=None):
    """First point of every occupied (scene, voxel), kept in input order; returns
    (keep (M,), point2voxel (N,), new_offset or None).  The reference leaves this step to
    its data pipeline; this is the definition the CUDA front end is held to."""
    import numpy as np
    b = batch.numpy().astype(np.int64)
    g = grid_coord.numpy().astype(np.int64)
    key = (b << 48) | (g[:, 0] << 32) | (g[:, 1] << 16) | g[:, 2]
    _, first, inverse = np.unique(key, return_index=True, return_inverse=True)
    keep = np.sort(first)
    rank = np.empty(key.shape[0], dtype=np.int64)
    rank[keep] = np.arange(keep.shape[0])
    point2voxel = rank[first[inverse.reshape(-1)]]
    new_offset = None
    if offset is not None:
        new_offset = torch.from_numpy(np.searchsorted(keep, offset.numpy(), side="left").astype(np.int64))
    return torch.from_numpy(keep), torch.from_numpy(point2voxel), new_offset


def adaptive_depth(grid_coord):
    """model.py:98-101."""
    return int(grid_coord.max()).bit_length()


def serialization(grid_coord, batch, orders=ORDERS, depth=None, perm=None):
    """Returns (code, order, inverse, depth), each (k, N) int64.

    Ties are ordered by original index (the reference calls an unstable
    ``argsort``; the stable order is the canonical representative).
    ``perm`` is the row permutation the reference draws with ``torch.randperm``
    when ``shuffle_orders`` is set (model.py:128-132).
    """
    if depth is None:
        depth = adaptive_depth(grid_coord)
    g = grid_coord.cpu().numpy()
    b = batch.cpu().numpy()
    code = np.stack([cenc.encode(g, b, depth, o) for o in orders])
    order = np.stack([cenc.argsort_stable(c) for c in code])
    inverse = np.stack([cenc.inverse(o) for o in order])
    code, order, inverse = (torch.from_numpy(a) for a in (code, order, inverse))
    if perm is not None:
        code, order, inverse = code[perm], order[perm], inverse[perm]
    return code, order, inverse, depth


# --------------------------------------------------------------------------- #
# model.py:382-438  SerializedAttention.get_padding_and_inverse
# --------------------------------------------------------------------------- #
def pad_plan(offset, K):
    """Returns (pad int64 (N_pad,), unpad int64 (N,), cu_seqlens int32)."""
    counts = offset_to_counts(offset).tolist()
    pad, unpad, cu = [], [], []
    start, start_pad = 0, 0
    for n in counts:
        n_pad = n if n <= K else (n + K - 1) // K * K          # model.py:394-404
        idx = list(range(n))
        if n_pad != n:
            r = n % K
            # the tail of the last patch re-uses the K - r ranks that precede
            # the last patch's real rows (model.py:412-422)
            idx += list(range(n - r - (K - r), n - r))
        pad += [start + i for i in idx]                         # model.py:423
        unpad += [start_pad + i for i in range(n)]              # model.py:411
        cu += list(range(start_pad, start_pad + n_pad, K))      # model.py:424-432
        start += n
        start_pad += n_pad
    cu.append(start_pad)
    return (torch.tensor(pad, dtype=torch.int64), torch.tensor(unpad, dtype=torch.int64),
            torch.tensor(cu, dtype=torch.int32))


def effective_patch(offset, patch_size_max):
    """model.py:441-444 (non-flash path)."""
    return min(int(offset_to_counts(offset).min()), patch_size_max)


# --------------------------------------------------------------------------- #
# model.py:440-490  SerializedAttention.forward, non-flash branch
# --------------------------------------------------------------------------- #
def rpe_bias(grid_coord_patches, table, pos_bnd):
    """model.py:297-316, 372-380: grid_coord_patches (N', K, 3) int -> (N', H, K, K)."""
    num = 2 * pos_bnd + 1
    rel = grid_coord_patches.unsqueeze(2) - grid_coord_patches.unsqueeze(1)
    idx = rel.clamp(-pos_bnd, pos_bnd) + pos_bnd + torch.arange(3) * num
    out = table.index_select(0, idx.reshape(-1).long()).view(idx.shape + (-1,)).sum(3)
    return out.permute(0, 3, 1, 2)


ATTENTION_CHUNK_BYTES = 1 << 30    # score tensors are built for this many bytes of patches at a time


def _patch_attention(q, k, v, scale, upcast_attention, upcast_softmax, bias=None):
    """softmax((q * scale) k^T [+ bias]) v over (P, H, K, d) tensors, model.py:467-474; patches are
    walked in groups so that the (P, H, K, K) score tensor stays bounded (same arithmetic)."""
    P, H, K, d = q.shape
    step = max(1, ATTENTION_CHUNK_BYTES // max(1, H * K * K * 4))
    outs = []
    for a in range(0, P, step):
        qq, kk, vv = q[a:a + step], k[a:a + step], v[a:a + step]
        if upcast_attention:
            qq, kk = qq.float(), kk.float()
        attn = (qq * scale) @ kk.transpose(-2, -1)              # model.py:467
        if bias is not None:
            attn = attn + bias[a:a + step]                      # model.py:468-469
        if upcast_softmax:
            attn = attn.float()
        attn = torch.softmax(attn, dim=-1).to(v.dtype)          # model.py:470-473
        outs.append(attn @ vv)
    return torch.cat(outs) if len(outs) > 1 else outs[0]


def attention(feat, w_qkv, b_qkv, w_proj, b_proj, order, inverse, offset, num_heads,
              patch_size_max, scale=None, upcast_attention=False, upcast_softmax=False, rpe=None,
              flash=False):
    """``rpe``: None or (grid_coord (N,3), table (3*num, H), pos_bnd).

    ``flash=True`` restates the grouping of the flash branch (model.py:475-483) in the
    feature dtype: the patch is ``patch_size_max`` itself and the sequences are the
    ``cu_seqlens`` segments, so a scene shorter than the patch is one short sequence.
    (The reference computes that branch in fp16 on a GPU library; the grouping is what
    is restated here, the arithmetic is the non-flash branch's.)"""
    N, C = feat.shape
    H = num_heads
    scale = scale or (C // H) ** -0.5
    K = patch_size_max if flash else effective_patch(offset, patch_size_max)
    pad, unpad, cu = pad_plan(offset, K)
    src = order[pad]                                            # model.py:452
    dst = unpad[inverse]                                        # model.py:453
    qkv = F.linear(feat, w_qkv, b_qkv)[src]                     # model.py:456
    if flash:
        assert rpe is None
        out = torch.empty(qkv.shape[0], C, dtype=qkv.dtype)
        cu = cu.tolist()
        lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
        i = 0
        while i < len(lens):
            # runs of equally long sequences (the full patches of a scene) go through one call
            j = i
            while j < len(lens) and lens[j] == lens[i]:
                j += 1
            L = lens[i]
            blk = qkv[cu[i]:cu[j]].reshape(j - i, L, 3, H, C // H).permute(2, 0, 3, 1, 4)
            o = _patch_attention(blk[0], blk[1], blk[2], scale, upcast_attention, upcast_softmax)
            out[cu[i]:cu[j]] = o.transpose(1, 2).reshape(-1, C)
            i = j
    else:
        q, k, v = qkv.reshape(-1, K, 3, H, C // H).permute(2, 0, 3, 1, 4).unbind(0)
        bias = None
        if rpe is not None:                                     # model.py:468-469
            grid_coord, table, pos_bnd = rpe
            bias = rpe_bias(grid_coord[src].reshape(-1, K, 3), table, pos_bnd)
        out = _patch_attention(q, k, v, scale, upcast_attention, upcast_softmax, bias)
        out = out.transpose(1, 2).reshape(-1, C)                # model.py:474
    out = out[dst]                                              # model.py:484
    return F.linear(out, w_proj, b_proj)                        # model.py:487


# --------------------------------------------------------------------------- #
# spconv.SubMConv3d as used at model.py:546-552 and :767-774.
# spconv is not part of the reference tree; the convention restated here is
# weight [C_out, kx, ky, kz, C_in], offset index ((dx+r)*k + (dy+r))*k + (dz+r),
# cross-correlation out[p] += W[d] . in[p + d].  Pinned against a dense conv3d.
# --------------------------------------------------------------------------- #
def kernel_map(indices, ksize):
    """indices (N,4) int (b,x,y,z) -> nbr (N, ksize**3) int64, -1 where absent.

    With duplicated rows the neighbour is the duplicate with the lowest index.
    """
    ind = indices.to(torch.int64)
    N = ind.shape[0]
    r = ksize // 2
    if N == 0:
        return torch.empty(0, ksize ** 3, dtype=torch.int64)
    ext = int(ind[:, 1:].max()) + 1 + 2 * r
    def lin(b, x, y, z):
        return ((b * ext + x) * ext + y) * ext + z
    keys = lin(ind[:, 0], ind[:, 1] + r, ind[:, 2] + r, ind[:, 3] + r)
    skeys, sidx = torch.sort(keys, stable=True)
    nbr = torch.full((N, ksize ** 3), -1, dtype=torch.int64)
    o = 0
    for dx in range(-r, r + 1):
        for dy in range(-r, r + 1):
            for dz in range(-r, r + 1):
                x, y, z = ind[:, 1] + dx, ind[:, 2] + dy, ind[:, 3] + dz
                ok = (x >= 0) & (y >= 0) & (z >= 0)
                q = lin(ind[:, 0], x + r, y + r, z + r)
                pos = torch.searchsorted(skeys, q).clamp(max=N - 1)
                hit = ok & (skeys[pos] == q)
                nbr[hit, o] = sidx[pos[hit]]
                o += 1
    return nbr


def subm_conv(feat, nbr, weight, bias=None):
    """feat (N,Cin); nbr (N,k^3); weight (Cout,k,k,k,Cin) -> (N,Cout) in feat.dtype."""
    N = feat.shape[0]
    cout, cin = weight.shape[0], weight.shape[-1]
    w = weight.reshape(cout, -1, cin).float()
    x = feat.float()
    out = torch.zeros(N, cout, dtype=torch.float32)
    for o in range(nbr.shape[1]):
        m = nbr[:, o] >= 0
        if m.any():
            out[m] += x[nbr[m, o]] @ w[:, o, :].t()
    if bias is not None:
        out += bias.float()
    return out.to(feat.dtype)


def sparse_indices(batch, grid_coord):
    """model.py:165-170."""
    return torch.cat([batch.unsqueeze(-1).int(), grid_coord.int()], dim=1).contiguous()


# --------------------------------------------------------------------------- #
# model.py:639-712  SerializedPooling.forward (bookkeeping part)
# --------------------------------------------------------------------------- #
def pooling_plan(code, depth, stride=2, perm=None):
    """code (k,N) int64 rows in the Point's current (shuffled) row order.

    Returns dict(cluster, indices, idx_ptr, head, code, order, inverse, depth,
    pooling_depth)."""
    pd = (math.ceil(stride) - 1).bit_length()
    if pd > depth:
        pd = 0                                                  # model.py:641-642
    c = code >> (pd * 3)                                        # model.py:652
    _, cluster, counts = torch.unique(c[0], sorted=True, return_inverse=True, return_counts=True)
    _, indices = torch.sort(cluster, stable=True)               # model.py:660
    idx_ptr = torch.cat([counts.new_zeros(1), torch.cumsum(counts, 0)])
    head = indices[idx_ptr[:-1]]                                # model.py:664
    pc = c[:, head]                                             # model.py:666
    order = torch.argsort(pc, stable=True)
    inverse = torch.zeros_like(order).scatter_(
        1, order, torch.arange(pc.shape[1]).repeat(pc.shape[0], 1))
    if perm is not None:
        pc, order, inverse = pc[perm], order[perm], inverse[perm]
    return dict(cluster=cluster, indices=indices, idx_ptr=idx_ptr, head=head, code=pc,
                order=order, inverse=inverse, depth=depth - pd, pooling_depth=pd)


def segment_reduce(src, idx_ptr, reduce):
    lengths = torch.diff(idx_ptr)
    return torch.segment_reduce(src, reduce, lengths=lengths, axis=0, unsafe=True)


def bn_eval(x, sd, prefix, eps=1e-3):
    """BatchNorm1d in eval mode (model.py:848: eps 1e-3)."""
    return F.batch_norm(x, sd[prefix + "running_mean"], sd[prefix + "running_var"],
                        sd[prefix + "weight"], sd[prefix + "bias"], False, 0.0, eps)


def ln(x, sd, prefix):
    return F.layer_norm(x, (x.shape[-1],), sd[prefix + "weight"], sd[prefix + "bias"], 1e-5)


# --------------------------------------------------------------------------- #
# Whole backbone, model.py:786-982, over a reference-layout state_dict
# --------------------------------------------------------------------------- #
DEFAULT_CFG = dict(
    in_channels=6, order=ORDERS, stride=(2, 2, 2, 2), enc_depths=(2, 2, 2, 6, 2),
    enc_channels=(32, 64, 128, 256, 512), enc_num_head=(2, 4, 8, 16, 32),
    enc_patch_size=(1024,) * 5, dec_depths=(2, 2, 2, 2), dec_channels=(64, 64, 128, 256),
    dec_num_head=(4, 4, 8, 16), dec_patch_size=(1024,) * 4, shuffle_orders=True, cls_mode=False,
)


class Level:
    """One resolution level of the hierarchy (what a reference Point holds)."""

    def __init__(self, **kw):
        self.__dict__.update(kw)
        self.nbr3 = None


def block(sd, p, lv, feat, heads, patch, order_index, conv_in=None, flash=False):
    """model.py:586-606 with pre_norm=True.

    ``conv_in``: what the xCPE convolution reads when it is not ``feat``.  The
    convolution runs on the Point's sparse tensor (model.py:233-236), and the
    unpooling adds the up-sampled features to ``feat`` only (model.py:746), so
    in the first block after an unpooling the convolution still sees the
    skip-projection alone while the residual uses the sum."""
    if lv.nbr3 is None:
        lv.nbr3 = kernel_map(sparse_indices(lv.batch, lv.grid_coord), 3)
    x = subm_conv(feat if conv_in is None else conv_in, lv.nbr3, sd[p + "cpe.0.weight"],
                  sd[p + "cpe.0.bias"])
    x = F.linear(x, sd[p + "cpe.1.weight"], sd[p + "cpe.1.bias"])
    feat = feat + ln(x, sd, p + "cpe.2.")
    x = ln(feat, sd, p + "norm1.0.")
    x = attention(x, sd[p + "attn.qkv.weight"], sd[p + "attn.qkv.bias"], sd[p + "attn.proj.weight"],
                  sd[p + "attn.proj.bias"], lv.order[order_index], lv.inverse[order_index],
                  lv.offset, heads, patch, flash=flash)
    feat = feat + x
    x = ln(feat, sd, p + "norm2.0.")
    x = F.linear(x, sd[p + "mlp.0.fc1.weight"], sd[p + "mlp.0.fc1.bias"])
    x = F.gelu(x)
    x = F.linear(x, sd[p + "mlp.0.fc2.weight"], sd[p + "mlp.0.fc2.bias"])
    return feat + x


def pool(sd, p, lv, feat, stride, shuffle):
    """model.py:639-712."""
    perm = torch.randperm(lv.code.shape[0]) if shuffle else None
    plan = pooling_plan(lv.code, lv.depth, stride, perm)
    x = F.linear(feat, sd[p + "proj.weight"], sd[p + "proj.bias"])
    x = segment_reduce(x[plan["indices"]], plan["idx_ptr"], "max")
    coord = segment_reduce(lv.coord[plan["indices"]], plan["idx_ptr"], "mean")
    batch = lv.batch[plan["head"]]
    new = Level(coord=coord, grid_coord=lv.grid_coord[plan["head"]] >> plan["pooling_depth"],
                batch=batch, offset=batch_to_offset(batch), code=plan["code"], order=plan["order"],
                inverse=plan["inverse"], depth=plan["depth"], cluster=plan["cluster"], parent=lv)
    x = F.gelu(bn_eval(x, sd, p + "norm.0."))
    return new, x


def unpool(sd, p, lv, feat, skip_feat):
    """model.py:739-750.  Returns (feat, skip branch alone)."""
    a = F.gelu(bn_eval(F.linear(feat, sd[p + "proj.0.weight"], sd[p + "proj.0.bias"]), sd, p + "proj.1."))
    b = F.gelu(bn_eval(F.linear(skip_feat, sd[p + "proj_skip.0.weight"], sd[p + "proj_skip.0.bias"]),
                       sd, p + "proj_skip.1."))
    return b + a[lv.cluster], b


def ptv3_forward(sd, data, cfg=None, return_levels=False, flash=False, taps=None):
    """Runs the backbone.  ``data``: feat, grid_coord, coord, offset.  Draws the
    same ``torch.randperm`` sequence as the reference (1 + one per pooling).
    ``flash``: the patch grouping of ``enable_flash=True`` (see ``attention``).
    ``taps``: a dict that receives the features after "embedding", every "enc.enc{s}"
    and every "dec.dec{s}"."""
    cfg = dict(DEFAULT_CFG, **(cfg or {}))
    tap = (lambda name, f: taps.__setitem__(name, f)) if taps is not None else (lambda name, f: None)
    orders = cfg["order"]
    offset = data["offset"].to(torch.int64)
    batch = offset_to_batch(offset)
    grid = data["grid_coord"]
    perm = None
    code, order, inverse, depth = serialization(grid, batch, orders)
    if cfg["shuffle_orders"]:
        perm = torch.randperm(len(orders))
        code, order, inverse = code[perm], order[perm], inverse[perm]
    lv = Level(coord=data["coord"], grid_coord=grid, batch=batch, offset=offset, code=code,
               order=order, inverse=inverse, depth=depth, cluster=None, parent=None)
    feat = data["feat"]
    # Embedding, model.py:766-783
    nbr5 = kernel_map(sparse_indices(batch, grid), 5)
    feat = subm_conv(feat, nbr5, sd["embedding.stem.conv.weight"], None)
    feat = F.gelu(bn_eval(feat, sd, "embedding.stem.norm."))
    tap("embedding", feat)
    levels, skips = [], []
    ns = len(cfg["enc_depths"])
    for s in range(ns):
        if s > 0:
            skips.append(feat)
            lv, feat = pool(sd, f"enc.enc{s}.down.", lv, feat, cfg["stride"][s - 1], cfg["shuffle_orders"])
        for i in range(cfg["enc_depths"][s]):
            feat = block(sd, f"enc.enc{s}.block{i}.", lv, feat, cfg["enc_num_head"][s],
                         cfg["enc_patch_size"][s], i % len(orders), flash=flash)
        tap(f"enc.enc{s}", feat)
        levels.append(lv)
    if not cfg["cls_mode"]:
        for s in reversed(range(ns - 1)):
            feat, stale = unpool(sd, f"dec.dec{s}.up.", lv, feat, skips[s])
            lv = lv.parent
            for i in range(cfg["dec_depths"][s]):
                feat = block(sd, f"dec.dec{s}.block{i}.", lv, feat, cfg["dec_num_head"][s],
                             cfg["dec_patch_size"][s], i % len(orders),
                             conv_in=stale if i == 0 else None, flash=flash)
            tap(f"dec.dec{s}", feat)
    if return_levels:
        return feat, levels
    return feat
