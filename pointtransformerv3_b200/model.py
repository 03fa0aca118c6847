"""Point Transformer V3 backbone with the reference's module names, constructor
arguments and state_dict layout (model.py:177-982).  Host code is PyTorch; the
point operators (serialization, patch attention, submanifold convolution,
pooling) call the CUDA library, dense Linear layers use torch's GEMM."""
import math
import sys
from collections import OrderedDict
from functools import partial

import torch
import torch.nn as nn

from . import _lib, ops
from . import sparse as spconv
from .point import AttrDict, Point, offset2bincount


class PointModule(nn.Module):
    """Modules derived from this class take and return a Point inside a
    PointSequential (model.py:177-183)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)


class PointSequential(PointModule):
    """Sequential container dispatching on module type (model.py:186-252): Point
    modules get the Point, sparse-convolution modules its sparse tensor, plain
    torch modules its feature matrix (mirrored into the sparse tensor)."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        if len(args) == 1 and isinstance(args[0], OrderedDict):
            for key, module in args[0].items():
                self.add_module(key, module)
        else:
            for idx, module in enumerate(args):
                self.add_module(str(idx), module)
        for name, module in kwargs.items():
            if name in self._modules:
                raise ValueError("name exists.")
            self.add_module(name, module)

    def __getitem__(self, idx):
        if not (-len(self) <= idx < len(self)):
            raise IndexError("index {} is out of range".format(idx))
        if idx < 0:
            idx += len(self)
        return list(self._modules.values())[idx]

    def __len__(self):
        return len(self._modules)

    def add(self, module, name=None):
        if name is None:
            name = str(len(self._modules))
            if name in self._modules:
                raise KeyError("name exists")
        self.add_module(name, module)

    def forward(self, input):
        for module in self._modules.values():
            if isinstance(module, PointModule):
                input = module(input)
            elif spconv.modules.is_spconv_module(module):
                if isinstance(input, Point):
                    input.sparse_conv_feat = module(input.sparse_conv_feat)
                    input.feat = input.sparse_conv_feat.features
                else:
                    input = module(input)
            else:
                if isinstance(input, Point):
                    input.feat = module(input.feat)
                    if "sparse_conv_feat" in input.keys():
                        input.sparse_conv_feat = input.sparse_conv_feat.replace_feature(input.feat)
                elif isinstance(input, spconv.SparseConvTensor):
                    if input.indices.shape[0] != 0:
                        input = input.replace_feature(module(input.features))
                else:
                    input = module(input)
        return input


class PDNorm(PointModule):
    """Per-dataset normalisation with optional context modulation (model.py:255-294):
    one norm layer per entry of ``conditions``, selected by ``point.condition``; with
    ``adaptive`` the result is scaled and shifted by a projection of ``point.context``.
    With ``decouple=False`` a single norm layer is shared (the reference stores the
    layer class itself there, which cannot be applied to a tensor)."""

    def __init__(self, num_features, norm_layer, context_channels=256,
                 conditions=("ScanNet", "S3DIS", "Structured3D"), decouple=True, adaptive=False):
        super().__init__()
        self.conditions = conditions
        self.decouple = decouple
        self.adaptive = adaptive
        if decouple:
            self.norm = nn.ModuleList([norm_layer(num_features) for _ in conditions])
        else:
            self.norm = norm_layer(num_features)
        if adaptive:
            self.modulation = nn.Sequential(nn.SiLU(), nn.Linear(context_channels, 2 * num_features, bias=True))

    def forward(self, point):
        assert {"feat", "condition"}.issubset(point.keys())
        condition = point.condition if isinstance(point.condition, str) else point.condition[0]
        if self.decouple:
            assert condition in self.conditions
            norm = self.norm[self.conditions.index(condition)]
        else:
            norm = self.norm
        feat = norm(point.feat)
        if self.adaptive:
            assert "context" in point.keys()
            shift, scale = self.modulation(point.context).chunk(2, dim=1)
            feat = feat * (1.0 + scale) + shift
        point.feat = feat
        return point


def _bn_eval_affine(bn):
    """Per-channel (scale, shift) of a BatchNorm1d in eval mode, fp32.  Cached on
    the module and recomputed when a parameter or buffer was modified or moved."""
    tensors = (bn.weight, bn.bias, bn.running_mean, bn.running_var)
    key = tuple((t._version, t.data_ptr(), t.dtype) if t is not None else None for t in tensors)
    cached = bn.__dict__.get("_ptv3_affine")
    if cached is not None and cached[0] == key:
        return cached[1], cached[2]
    w = bn.weight.float() if bn.weight is not None else torch.ones_like(bn.running_var)
    b = bn.bias.float() if bn.bias is not None else torch.zeros_like(bn.running_var)
    scale = (w * torch.rsqrt(bn.running_var.float() + bn.eps)).contiguous()
    shift = (b - bn.running_mean.float() * scale).contiguous()
    bn.__dict__["_ptv3_affine"] = (key, scale, shift)
    return scale, shift


def _is_bn_gelu(norm, act):
    """True when (norm, act) is the BatchNorm1d(eval) + exact GELU pair the fused
    pooling kernels implement."""
    if norm is None or act is None or len(norm) != 1 or len(act) != 1:
        return False
    n, a = norm[0], act[0]
    return (type(n) is nn.BatchNorm1d and not n.training and n.track_running_stats
            and type(a) is nn.GELU and getattr(a, "approximate", "none") == "none")


class RPE(nn.Module):
    """Relative position bias table (model.py:297-316).  The lookup and the sum
    over the three axes happen inside the attention kernel; ``forward`` keeps the
    reference's tensor form for stand-alone use."""

    def __init__(self, patch_size, num_heads):
        super().__init__()
        self.patch_size = patch_size
        self.num_heads = num_heads
        self.pos_bnd = int((4 * patch_size) ** (1 / 3) * 2)
        self.rpe_num = 2 * self.pos_bnd + 1
        self.rpe_table = nn.Parameter(torch.zeros(3 * self.rpe_num, num_heads))
        nn.init.trunc_normal_(self.rpe_table, std=0.02)

    def forward(self, coord):
        idx = (coord.clamp(-self.pos_bnd, self.pos_bnd) + self.pos_bnd
               + torch.arange(3, device=coord.device) * self.rpe_num)
        out = self.rpe_table.index_select(0, idx.reshape(-1))
        out = out.view(idx.shape + (-1,)).sum(3)
        return out.permute(0, 3, 1, 2)


class SerializedAttention(PointModule):
    """Multi-head self-attention inside patches of a serialized order
    (model.py:319-490).  Both settings of ``enable_flash`` run the same CUDA
    kernel; the flag keeps the reference's patch-size rule: off -> patch =
    min(smallest scene, patch_size) re-evaluated per call (model.py:441-444),
    on -> patch = patch_size with shorter scenes as one short sequence."""

    def __init__(self, channels, num_heads, patch_size, qkv_bias=True, qk_scale=None, attn_drop=0.0,
                 proj_drop=0.0, order_index=0, enable_rpe=False, enable_flash=True,
                 upcast_attention=True, upcast_softmax=True):
        super().__init__()
        assert channels % num_heads == 0
        self.channels = channels
        self.num_heads = num_heads
        self.scale = qk_scale or (channels // num_heads) ** -0.5
        self.order_index = order_index
        self.upcast_attention = upcast_attention
        self.upcast_softmax = upcast_softmax
        self.enable_rpe = enable_rpe
        self.enable_flash = enable_flash
        if enable_flash:
            assert enable_rpe is False, "Set enable_rpe to False when enable Flash Attention"
            assert upcast_attention is False, "Set upcast_attention to False when enable Flash Attention"
            assert upcast_softmax is False, "Set upcast_softmax to False when enable Flash Attention"
            self.patch_size = patch_size
        else:
            self.patch_size_max = patch_size
            self.patch_size = 0
        self.attn_drop = attn_drop
        self.qkv = nn.Linear(channels, channels * 3, bias=qkv_bias)
        self.proj = nn.Linear(channels, channels)
        self.proj_drop = nn.Dropout(proj_drop)
        self.rpe = RPE(patch_size, num_heads) if self.enable_rpe else None
        self.algo = 0

    @torch.no_grad()
    def get_padding_and_inverse(self, point):
        """model.py:382-438; cached in the Point under the reference's keys.

        The reference reuses whatever plan is cached, also when a later block of the same
        level has another patch size (encoder and decoder patch sizes may differ), which
        there groups rows wrongly.  Here the patch size a plan was made for is kept beside
        it and the plan is rebuilt when this module's differs."""
        if (not {"pad", "unpad", "cu_seqlens_key"}.issubset(point.keys())
                or point.get("_pad_patch", self.patch_size) != self.patch_size):
            pad, unpad, cu = ops.pad_plan(point.offset, point.host_counts(), self.patch_size,
                                          point.device_status())
            point.check_status("ptv3_pad_plan")
            point["pad"], point["unpad"], point["cu_seqlens_key"] = pad, unpad, cu
            point["_pad_patch"] = self.patch_size
        return point["pad"], point["unpad"], point["cu_seqlens_key"]

    def core(self, point, qkv):
        """Patch attention of an already projected (N, 3C) qkv matrix over
        ``point``'s serialized order; the output projection is not applied."""
        assert not self.training, "inference only"
        if not self.enable_flash:
            self.patch_size = min(min(point.host_counts()), self.patch_size_max)
        pad, unpad, cu_seqlens = self.get_padding_and_inverse(point)
        if self.enable_rpe:
            return ops.attention_rpe(qkv, point.serialized_order[self.order_index], pad, unpad, cu_seqlens,
                                     point.grid_coord, self.rpe.rpe_table, self.rpe.pos_bnd, self.num_heads,
                                     self.patch_size, self.scale)
        return ops.attention(qkv, point.serialized_order[self.order_index], pad, unpad, cu_seqlens,
                             self.num_heads, self.patch_size, self.scale, self.algo,
                             status=point.device_status())

    def attend(self, point, feat):
        """qkv projection, patch attention and output projection of ``feat``."""
        return self.proj_drop(self.proj(self.core(point, self.qkv(feat))))

    def forward(self, point):
        point.feat = self.attend(point, point.feat)
        return point


class MLP(nn.Module):
    """model.py:493-516."""

    def __init__(self, in_channels, hidden_channels=None, out_channels=None, act_layer=nn.GELU, drop=0.0):
        super().__init__()
        out_channels = out_channels or in_channels
        hidden_channels = hidden_channels or in_channels
        self.fc1 = nn.Linear(in_channels, hidden_channels)
        self.act = act_layer()
        self.fc2 = nn.Linear(hidden_channels, out_channels)
        self.drop = nn.Dropout(drop)

    def forward(self, x):
        return self.drop(self.fc2(self.drop(self.act(self.fc1(x)))))


class Block(PointModule):
    """xCPE convolution + attention + MLP with residuals (model.py:519-606)."""

    def __init__(self, channels, num_heads, patch_size=48, mlp_ratio=4.0, qkv_bias=True, qk_scale=None,
                 attn_drop=0.0, proj_drop=0.0, drop_path=0.0, norm_layer=nn.LayerNorm, act_layer=nn.GELU,
                 pre_norm=True, order_index=0, cpe_indice_key=None, enable_rpe=False, enable_flash=True,
                 upcast_attention=True, upcast_softmax=True):
        super().__init__()
        self.channels = channels
        self.pre_norm = pre_norm
        self.cpe = PointSequential(
            spconv.SubMConv3d(channels, channels, kernel_size=3, bias=True, indice_key=cpe_indice_key),
            nn.Linear(channels, channels),
            norm_layer(channels),
        )
        self.norm1 = PointSequential(norm_layer(channels))
        self.attn = SerializedAttention(
            channels=channels, patch_size=patch_size, num_heads=num_heads, qkv_bias=qkv_bias,
            qk_scale=qk_scale, attn_drop=attn_drop, proj_drop=proj_drop, order_index=order_index,
            enable_rpe=enable_rpe, enable_flash=enable_flash, upcast_attention=upcast_attention,
            upcast_softmax=upcast_softmax)
        self.norm2 = PointSequential(norm_layer(channels))
        self.mlp = PointSequential(MLP(in_channels=channels, hidden_channels=int(channels * mlp_ratio),
                                       out_channels=channels, act_layer=act_layer, drop=proj_drop))
        # stochastic depth is the identity at inference; the rate is kept for bookkeeping
        self.drop_path_rate = drop_path
        self.drop_path = PointSequential(nn.Identity())

    def _fusable(self, point):
        """The fused path covers the reference configuration: pre-norm, plain
        affine LayerNorms, exact GELU, fp32 or bf16 features."""
        def plain_ln(m):
            return type(m) is nn.LayerNorm and m.elementwise_affine and m.bias is not None
        mlp = self.mlp[0] if len(self.mlp) == 1 else None
        return (self.pre_norm and len(self.cpe) == 3 and isinstance(self.cpe[0], spconv.SubMConv3d)
                and type(self.cpe[1]) is nn.Linear and plain_ln(self.cpe[2])
                and len(self.norm1) == 1 and plain_ln(self.norm1[0])
                and len(self.norm2) == 1 and plain_ln(self.norm2[0])
                and type(mlp) is MLP and type(mlp.act) is nn.GELU
                and getattr(mlp.act, "approximate", "none") == "none"
                and point.feat.dtype in (torch.float32, torch.bfloat16)
                and "sparse_conv_feat" in point.keys())

    def _native_args(self, dt, device):
        """The argument block of ptv3_block_fwd with this block's parameters filled
        in.  It is rebuilt whenever a parameter object or its storage changed; the
        check walks the submodules' parameter dicts directly, which costs a few
        microseconds instead of the attribute lookups of a rebuild."""
        cached = self.__dict__.get("_ptv3_block_args")
        if cached is not None:
            holders, params, ptrs, a = cached
            for (owner, name), p, ptr in zip(holders, params, ptrs):
                if owner[name] is not p or p.data_ptr() != ptr:
                    break
            else:
                if params[0].dtype == dt and params[0].device == device:
                    a.attention_algo, a.scale = self.attn.algo, self.attn.scale
                    return a
        conv, lin, attn, mlp = self.cpe[0], self.cpe[1], self.attn, self.mlp[0]
        names = ("conv_weight", "conv_bias", "cpe_w", "cpe_b", "cpe_ln_w", "cpe_ln_b", "n1_w", "n1_b", "qkv_w",
                 "qkv_b", "proj_w", "proj_b", "n2_w", "n2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b")
        owners = (conv, conv, lin, lin, self.cpe[2], self.cpe[2], self.norm1[0], self.norm1[0], attn.qkv, attn.qkv,
                  attn.proj, attn.proj, self.norm2[0], self.norm2[0], mlp.fc1, mlp.fc1, mlp.fc2, mlp.fc2)
        holders = tuple((m._parameters, "weight" if i % 2 == 0 else "bias") for i, m in enumerate(owners))
        params = tuple(owner[name] for owner, name in holders)
        if any(p is None or p.dtype != dt or p.device != device or not p.is_contiguous() for p in params):
            self.__dict__.pop("_ptv3_block_args", None)
            return None
        ptrs = tuple(p.data_ptr() for p in params)
        a = _lib.BlockArgs()
        a.channels, a.heads, a.hidden = self.channels, attn.num_heads, mlp.fc1.out_features
        a.dtype = _lib.DTYPE_IDS[dt]
        a.cpe_ln_eps, a.n1_eps, a.n2_eps = self.cpe[2].eps, self.norm1[0].eps, self.norm2[0].eps
        for name, ptr in zip(names, ptrs):
            setattr(a, name, ptr)
        self.__dict__["_ptv3_block_args"] = (holders, params, ptrs, a)
        a.attention_algo, a.scale = attn.algo, attn.scale
        return a

    def _native_static_ok(self, dt):
        """Shape conditions of the single-call path that do not depend on the input."""
        key = ("_ptv3_native_ok", dt)
        ok = self.__dict__.get(key)
        if ok is None:
            attn, mlp, conv = self.attn, self.mlp[0], self.cpe[0]
            ok = (conv.kernel_size == 3 and conv.in_channels == self.channels
                  and conv.out_channels == self.channels and mlp.fc2.out_features == self.channels
                  and mlp.fc1.in_features == self.channels
                  and ops.block_supported(self.channels, attn.num_heads, mlp.fc1.out_features, dt))
            self.__dict__[key] = ok
        return ok

    def _forward_native(self, point):
        """The whole block queued by one C call (ptv3_block_fwd); None when the
        configuration is outside what that entry point covers."""
        shortcut, sparse = point.feat, point.sparse_conv_feat
        attn = self.attn
        dt = shortcut.dtype
        if ops.TIMERS is not None or attn.enable_rpe or not self._native_static_ok(dt):
            return None
        args = self._native_args(dt, shortcut.device)
        if args is None:
            return None
        if not attn.enable_flash:
            attn.patch_size = min(min(point.host_counts()), attn.patch_size_max)
        pad, unpad, cu_seqlens = attn.get_padding_and_inverse(point)
        feat = ops.block(args, sparse.features, shortcut, self.cpe[0].geometry(sparse),
                         {"order": point.serialized_order[attn.order_index], "pad": pad, "unpad": unpad,
                          "cu_seqlens": cu_seqlens, "max_seqlen": attn.patch_size}, point.device_status())
        point.check_status("ptv3_block_fwd")
        point.feat = feat
        point.sparse_conv_feat = sparse.replace_feature(feat)
        return point

    def _forward_fused(self, point):
        """Same arithmetic as the generic path with the LayerNorms and residual
        additions done by the fused row kernel (three launches instead of eight);
        bf16 blocks go through one C call (the per-operator path below is kept for
        fp32 and for per-operator timing)."""
        done = self._forward_native(point)
        if done is not None:
            return done
        shortcut = point.feat
        sparse = point.sparse_conv_feat
        status = point.device_status()
        C, dt = self.channels, shortcut.dtype
        attn, lin = self.attn, self.cpe[1]
        # the convolution reads the sparse tensor's features, which differ from
        # `feat` right after an unpooling (model.py:233-236, 744-746)
        x = self.cpe[0](sparse).features
        if (lin.bias is not None and attn.qkv.bias is not None and ops.linear_supported(C, C, True, dt)
                and ops.linear_supported(C, 3 * C, False, dt)):
            # Linear layers with their LayerNorm / residual glue in the GEMM epilogue (tcgen05)
            feat, normed = ops.linear_ln(x, lin.weight, lin.bias, shortcut, self.cpe[2], self.norm1[0], status)
            x = attn.core(point, ops.linear(normed, attn.qkv.weight, attn.qkv.bias, status))
            feat, normed = ops.linear_ln(x, attn.proj.weight, attn.proj.bias, feat, None, self.norm2[0], status)
            point.check_status("tcgen05 linear layers")
        else:
            # wide channels: the streamed-weight tensor-core Linear (bf16) or torch's (fp32), with
            # the LayerNorm / residual glue in the fused row kernel
            feat, normed = ops.add_layernorm(_linear_op(x, lin, status), shortcut, self.cpe[2], self.norm1[0])
            x = _linear_op(attn.core(point, _linear_op(normed, attn.qkv, status)), attn.proj, status)
            feat, normed = ops.add_layernorm(x, feat, None, self.norm2[0])
        mlp = self.mlp[0]
        if (mlp.fc1.bias is not None and mlp.fc2.bias is not None
                and ops.mlp_supported(mlp.fc1.in_features, mlp.fc1.out_features, normed.dtype)
                and mlp.fc2.out_features == mlp.fc1.in_features):
            # both GEMMs, GELU and the residual in one tcgen05 kernel
            feat = ops.mlp(normed, mlp.fc1.weight, mlp.fc1.bias, mlp.fc2.weight, mlp.fc2.bias, feat,
                           point.device_status())
            point.check_status("ptv3_mlp_fwd")
        elif (mlp.fc1.bias is not None and mlp.fc2.bias is not None and normed.dtype == torch.bfloat16
              and ops.gemm_supported(mlp.fc1.in_features, mlp.fc1.out_features, normed.dtype)
              and ops.gemm_supported(mlp.fc2.in_features, mlp.fc2.out_features, normed.dtype)):
            # bias + GELU and bias + residual in the epilogues of the two Linear kernels
            hidden = ops.gemm(normed, mlp.fc1.weight, mlp.fc1.bias, None, True, status)
            feat = ops.gemm(hidden, mlp.fc2.weight, mlp.fc2.bias, feat, False, status)
            point.check_status("ptv3_gemm_fwd")
        else:
            x = mlp(normed)
            feat, _ = ops.add_layernorm(x, feat, None, None)
        point.feat = feat
        point.sparse_conv_feat = sparse.replace_feature(feat)
        return point

    def forward(self, point):
        assert not self.training, "inference only"
        if self._fusable(point):
            return self._forward_fused(point)
        shortcut = point.feat
        point = self.cpe(point)
        point.feat = shortcut + point.feat
        shortcut = point.feat
        if self.pre_norm:
            point = self.norm1(point)
        point = self.drop_path(self.attn(point))
        point.feat = shortcut + point.feat
        if not self.pre_norm:
            point = self.norm1(point)
        shortcut = point.feat
        if self.pre_norm:
            point = self.norm2(point)
        point = self.drop_path(self.mlp(point))
        point.feat = shortcut + point.feat
        if not self.pre_norm:
            point = self.norm2(point)
        point.sparse_conv_feat = point.sparse_conv_feat.replace_feature(point.feat)
        return point


class SerializedPooling(PointModule):
    """Pools the points that share a parent cell of the serialization grid
    (model.py:609-712)."""

    def __init__(self, in_channels, out_channels, stride=2, norm_layer=None, act_layer=None, reduce="max",
                 shuffle_orders=True, traceable=True):
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        assert stride == 2 ** (math.ceil(stride) - 1).bit_length()
        self.stride = stride
        assert reduce in ["sum", "mean", "min", "max"]
        self.reduce = reduce
        self.shuffle_orders = shuffle_orders
        self.traceable = traceable
        self.proj = nn.Linear(in_channels, out_channels)
        self.norm = PointSequential(norm_layer(out_channels)) if norm_layer is not None else None
        self.act = PointSequential(act_layer()) if act_layer is not None else None

    def plan(self, point):
        """Index side of the pooling (model.py:640-680, 690-695): clusters, pooled
        codes/orders/inverses, grid coordinates and scene ids of the coarse level,
        returned as a Point without features.  Draws the order shuffle.  One host
        read (the size of the coarse level)."""
        pooling_depth = (math.ceil(self.stride) - 1).bit_length()
        if pooling_depth > point.serialized_depth:
            pooling_depth = 0
        assert {"serialized_code", "serialized_order", "serialized_inverse", "serialized_depth"}.issubset(
            point.keys()), "Run point.serialization() point cloud before SerializedPooling"
        k = point.serialized_code.shape[0]
        perm = torch.randperm(k).tolist() if self.shuffle_orders else None
        plan = ops.pool_plan(point.serialized_code, point.serialized_order, point.grid_coord, point.batch,
                             len(point.offset), pooling_depth, perm, point.device_status())
        child = Point(AttrDict(
            grid_coord=plan["grid_coord"],
            serialized_code=plan["code"],
            serialized_order=plan["order"],
            serialized_inverse=plan["inverse"],
            serialized_depth=point.serialized_depth - pooling_depth,
            batch=plan["batch"],
            offset=plan["offset"],
        ))
        child["_counts"] = plan["counts"]
        child["_status"] = point.device_status()
        child["_defer_status"] = point.get("_defer_status", False)
        child["_idx_ptr"] = plan["idx_ptr"]
        child["_cluster"] = plan["cluster"]
        if "_shape_pad" in point.keys():
            # max(coord >> d) == max(coord) >> d, so the coarse sparse shape follows
            # from the fine one without reading the device (model.py:162-164)
            pad = point["_shape_pad"]
            child["sparse_shape"] = [((v - pad) >> pooling_depth) + pad for v in point.sparse_shape]
            child["_shape_pad"] = pad
        return child

    def forward(self, point):
        assert not self.training, "inference only"
        child = point.pop("_pooled_child", None)
        if child is None:
            child = self.plan(point)
        fused = _is_bn_gelu(self.norm, self.act)
        scale = shift = None
        if fused:
            scale, shift = _bn_eval_affine(self.norm[0])
        src_coord = point.coord if "coord" in point.keys() else None
        if _single_call_ok(point.feat, self.proj):
            # projection and reduction queued by one C call
            feat, coord = ops.pool_stage(point.feat, self.proj.weight, self.proj.bias, src_coord,
                                         point.serialized_order[0], child.pop("_idx_ptr"), scale, shift,
                                         self.reduce, point.device_status())
            point.check_status("ptv3_pool_stage_fwd")
        else:
            feat, coord = ops.pool(_linear_op(point.feat, self.proj, point.device_status()), src_coord,
                                   point.serialized_order[0], child.pop("_idx_ptr"), scale, shift, self.reduce)
        cluster = child.pop("_cluster")
        child["feat"] = feat
        if coord is not None:
            child["coord"] = coord
        if "condition" in point.keys():
            child["condition"] = point.condition
        if "context" in point.keys():
            child["context"] = point.context
        if self.traceable:
            child["pooling_inverse"] = cluster
            child["pooling_parent"] = point
        point = child
        if not fused:
            if self.norm is not None:
                point = self.norm(point)
            if self.act is not None:
                point = self.act(point)
        point.sparsify()
        return point


class SerializedUnpooling(PointModule):
    """Projects the coarse level and its skip connection and adds the
    up-sampled coarse features to the parent level (model.py:715-750)."""

    def __init__(self, in_channels, skip_channels, out_channels, norm_layer=None, act_layer=None,
                 traceable=False):
        super().__init__()
        self.proj = PointSequential(nn.Linear(in_channels, out_channels))
        self.proj_skip = PointSequential(nn.Linear(skip_channels, out_channels))
        if norm_layer is not None:
            self.proj.add(norm_layer(out_channels))
            self.proj_skip.add(norm_layer(out_channels))
        if act_layer is not None:
            self.proj.add(act_layer())
            self.proj_skip.add(act_layer())
        self.traceable = traceable

    def _fusable(self):
        def ok(seq):
            return (len(seq) == 3 and type(seq[1]) is nn.BatchNorm1d and not seq[1].training
                    and type(seq[2]) is nn.GELU and getattr(seq[2], "approximate", "none") == "none")
        return ok(self.proj) and ok(self.proj_skip)

    def forward(self, point):
        assert not self.training, "inference only"
        assert "pooling_parent" in point.keys()
        assert "pooling_inverse" in point.keys()
        parent = point.pop("pooling_parent")
        inverse = point.pop("pooling_inverse")
        if self._fusable():
            cs, cb = _bn_eval_affine(self.proj[1])
            ss, sb = _bn_eval_affine(self.proj_skip[1])
            child_lin = None
            if (not self.traceable and _single_call_ok(point.feat, self.proj[0])
                    and _single_call_ok(parent.feat, self.proj_skip[0])):
                # both projections and the gather-add queued by one C call
                out, skip_act = ops.unpool_stage(parent.feat, point.feat, self.proj_skip[0].weight,
                                                 self.proj_skip[0].bias, self.proj[0].weight, self.proj[0].bias,
                                                 inverse, ss, sb, cs, cb, parent.device_status())
                parent.check_status("ptv3_unpool_stage_fwd")
            else:
                child_lin = _linear_op(point.feat, self.proj[0], parent.device_status())
                skip_lin = _linear_op(parent.feat, self.proj_skip[0], parent.device_status())
                out, skip_act = ops.unpool(skip_lin, child_lin, inverse, ss, sb, cs, cb)
            # the parent's sparse tensor keeps the skip branch alone: the reference
            # adds the up-sampled features to `feat` only (model.py:746), and the next
            # block's convolution reads the sparse tensor
            parent.feat = skip_act
            if "sparse_conv_feat" in parent.keys():
                parent.sparse_conv_feat = parent.sparse_conv_feat.replace_feature(skip_act)
            parent.feat = out
            if self.traceable:
                point.feat = torch.nn.functional.gelu(torch.nn.functional.batch_norm(
                    child_lin, self.proj[1].running_mean, self.proj[1].running_var, self.proj[1].weight,
                    self.proj[1].bias, False, 0.0, self.proj[1].eps))
        else:
            point = self.proj(point)
            parent = self.proj_skip(parent)
            parent.feat = parent.feat + point.feat[inverse]
        if self.traceable:
            parent["unpooling_parent"] = point
        return parent


class Embedding(PointModule):
    """Stem: 5x5x5 submanifold convolution + norm + activation (model.py:753-783)."""

    def __init__(self, in_channels, embed_channels, norm_layer=None, act_layer=None):
        super().__init__()
        self.in_channels = in_channels
        self.embed_channels = embed_channels
        self.stem = PointSequential(conv=spconv.SubMConv3d(in_channels, embed_channels, kernel_size=5,
                                                           padding=1, bias=False, indice_key="stem"))
        if norm_layer is not None:
            self.stem.add(norm_layer(embed_channels), name="norm")
        if act_layer is not None:
            self.stem.add(act_layer(), name="act")

    def forward(self, point):
        mods = list(self.stem._modules.values())
        conv = mods[0]
        # convolution + BatchNorm(eval) + GELU in one kernel when that is what the stem is
        if (len(mods) == 3 and isinstance(conv, spconv.SubMConv3d) and conv.uses_direct_path()
                and type(mods[1]) is nn.BatchNorm1d and not mods[1].training and mods[1].track_running_stats
                and type(mods[2]) is nn.GELU and getattr(mods[2], "approximate", "none") == "none"
                and "sparse_conv_feat" in point.keys()):
            scale, shift = _bn_eval_affine(mods[1])
            point.sparse_conv_feat = conv(point.sparse_conv_feat, scale, shift, True)
            point.feat = point.sparse_conv_feat.features
            return point
        return self.stem(point)


class PointTransformerV3(PointModule):
    """The backbone (model.py:786-982); constructor arguments as in the reference."""

    def __init__(self, in_channels=6, order=("z", "z-trans", "hilbert", "hilbert-trans"), stride=(2, 2, 2, 2),
                 enc_depths=(2, 2, 2, 6, 2), enc_channels=(32, 64, 128, 256, 512),
                 enc_num_head=(2, 4, 8, 16, 32), enc_patch_size=(1024, 1024, 1024, 1024, 1024),
                 dec_depths=(2, 2, 2, 2), dec_channels=(64, 64, 128, 256), dec_num_head=(4, 4, 8, 16),
                 dec_patch_size=(1024, 1024, 1024, 1024), mlp_ratio=4, qkv_bias=True, qk_scale=None,
                 attn_drop=0.0, proj_drop=0.0, drop_path=0.3, pre_norm=True, shuffle_orders=True,
                 enable_rpe=False, enable_flash=True, upcast_attention=False, upcast_softmax=False,
                 cls_mode=False, pdnorm_bn=False, pdnorm_ln=False, pdnorm_decouple=True,
                 pdnorm_adaptive=False, pdnorm_affine=True,
                 pdnorm_conditions=("ScanNet", "S3DIS", "Structured3D")):
        super().__init__()
        self.num_stages = len(enc_depths)
        self.order = [order] if isinstance(order, str) else order
        self.cls_mode = cls_mode
        # how many stages ahead of the features the pooling plans are made (see forward)
        self.plan_ahead = 2
        # True: forward() leaves the device status word unread (see forward)
        self.defer_status_check = False
        self.shuffle_orders = shuffle_orders
        assert self.num_stages == len(stride) + 1
        assert self.num_stages == len(enc_depths)
        assert self.num_stages == len(enc_channels)
        assert self.num_stages == len(enc_num_head)
        assert self.num_stages == len(enc_patch_size)
        assert self.cls_mode or self.num_stages == len(dec_depths) + 1
        assert self.cls_mode or self.num_stages == len(dec_channels) + 1
        assert self.cls_mode or self.num_stages == len(dec_num_head) + 1
        assert self.cls_mode or self.num_stages == len(dec_patch_size) + 1
        # per-dataset normalisation runs on torch's norm layers (the fused kernels take
        # over only for plain LayerNorm / BatchNorm1d, i.e. when these flags are off)
        if pdnorm_bn:
            bn_layer = partial(PDNorm, norm_layer=partial(nn.BatchNorm1d, eps=1e-3, momentum=0.01,
                                                          affine=pdnorm_affine),
                               conditions=pdnorm_conditions, decouple=pdnorm_decouple, adaptive=pdnorm_adaptive)
        else:
            bn_layer = partial(nn.BatchNorm1d, eps=1e-3, momentum=0.01)
        if pdnorm_ln:
            ln_layer = partial(PDNorm, norm_layer=partial(nn.LayerNorm, elementwise_affine=pdnorm_affine),
                               conditions=pdnorm_conditions, decouple=pdnorm_decouple, adaptive=pdnorm_adaptive)
        else:
            ln_layer = nn.LayerNorm
        act_layer = nn.GELU

        self.embedding = Embedding(in_channels=in_channels, embed_channels=enc_channels[0],
                                   norm_layer=bn_layer, act_layer=act_layer)
        enc_drop_path = [x.item() for x in torch.linspace(0, drop_path, sum(enc_depths))]
        self.enc = PointSequential()
        for s in range(self.num_stages):
            enc_drop_path_ = enc_drop_path[sum(enc_depths[:s]): sum(enc_depths[: s + 1])]
            enc = PointSequential()
            if s > 0:
                enc.add(SerializedPooling(in_channels=enc_channels[s - 1], out_channels=enc_channels[s],
                                          stride=stride[s - 1], norm_layer=bn_layer, act_layer=act_layer),
                        name="down")
            for i in range(enc_depths[s]):
                enc.add(Block(channels=enc_channels[s], num_heads=enc_num_head[s],
                              patch_size=enc_patch_size[s], mlp_ratio=mlp_ratio, qkv_bias=qkv_bias,
                              qk_scale=qk_scale, attn_drop=attn_drop, proj_drop=proj_drop,
                              drop_path=enc_drop_path_[i], norm_layer=ln_layer, act_layer=act_layer,
                              pre_norm=pre_norm, order_index=i % len(self.order),
                              cpe_indice_key=f"stage{s}", enable_rpe=enable_rpe, enable_flash=enable_flash,
                              upcast_attention=upcast_attention, upcast_softmax=upcast_softmax),
                        name=f"block{i}")
            if len(enc) != 0:
                self.enc.add(module=enc, name=f"enc{s}")

        if not self.cls_mode:
            dec_drop_path = [x.item() for x in torch.linspace(0, drop_path, sum(dec_depths))]
            self.dec = PointSequential()
            dec_channels = list(dec_channels) + [enc_channels[-1]]
            for s in reversed(range(self.num_stages - 1)):
                dec_drop_path_ = dec_drop_path[sum(dec_depths[:s]): sum(dec_depths[: s + 1])]
                dec_drop_path_.reverse()
                dec = PointSequential()
                dec.add(SerializedUnpooling(in_channels=dec_channels[s + 1], skip_channels=enc_channels[s],
                                            out_channels=dec_channels[s], norm_layer=bn_layer,
                                            act_layer=act_layer), name="up")
                for i in range(dec_depths[s]):
                    dec.add(Block(channels=dec_channels[s], num_heads=dec_num_head[s],
                                  patch_size=dec_patch_size[s], mlp_ratio=mlp_ratio, qkv_bias=qkv_bias,
                                  qk_scale=qk_scale, attn_drop=attn_drop, proj_drop=proj_drop,
                                  drop_path=dec_drop_path_[i], norm_layer=ln_layer, act_layer=act_layer,
                                  pre_norm=pre_norm, order_index=i % len(self.order),
                                  cpe_indice_key=f"stage{s}", enable_rpe=enable_rpe,
                                  enable_flash=enable_flash, upcast_attention=upcast_attention,
                                  upcast_softmax=upcast_softmax), name=f"block{i}")
                self.dec.add(module=dec, name=f"dec{s}")

    def _side_stream(self, device):
        streams = self.__dict__.setdefault("_ptv3_side_streams", {})
        if device not in streams:
            # high priority: the plan kernels are tiny and must not queue behind the blocks of a
            # feature kernel that fills the GPU
            streams[device] = torch.cuda.Stream(device=device, priority=-1)
        return streams[device]

    def forward(self, data_dict):
        """data_dict: ``feat``, ``grid_coord`` (or ``coord`` + ``grid_size``) and
        ``offset`` or ``batch``; returns the Point of the finest level.

        Extensions, all optional.  ``serialization_depth`` fixes the depth of the
        codes instead of deriving it from this batch's largest coordinate (needed
        when one logical batch is split over several processes).  ``offset_host``
        (the cumulative scene sizes as a Python list or CPU tensor) together with
        ``sparse_shape`` (largest grid coordinate per axis + 96) and
        ``serialization_depth`` lets a caller that knows these on the host skip the one
        device read at the start of the pass; a caller that streams batches from host
        memory should do so, because that read is a small device-to-host copy which waits
        behind any large copy the same engine is busy with (the previous batch's output).  With
        ``self.defer_status_check = True`` the device status word is not read at
        the end either; the caller checks ``point.check_status(force=True)`` (or reads
        ``point["_status"]`` together with the output) when it next needs the host to
        wait.  Passes queued back to back then overlap: serialization and the pooling
        plans of one pass run on the planning stream while the main stream still holds
        the features of the pass before it (benchmark batch: 8.55 ms per pass with the
        status read at the end of every pass, 8.2 ms with it deferred)."""
        point = Point(data_dict)
        depth = point.pop("serialization_depth", None)
        host_offset = point.pop("offset_host", None)
        if host_offset is not None and "_counts" not in point.keys():
            off = [0] + [int(v) for v in (host_offset.tolist() if hasattr(host_offset, "tolist") else host_offset)]
            point["_counts"] = [off[i + 1] - off[i] for i in range(len(off) - 1)]
        status = point.device_status()
        point["_defer_status"] = True
        feat_dtype = point.feat.dtype
        # -- Schedule.  Serialization and the pooling plans need only coordinates.  They run on a
        #    second, high-priority stream: a plan has one host read (its size) and a few dozen small
        #    launches, and is made two stages ahead of the features (level 1 while the stem runs,
        #    level s + 2 while stage s runs), so that the host reads never wait behind, and never hold
        #    up, the feature kernels.  Nothing on that stream depends on the main stream beyond the
        #    inputs, so with deferred status checks the planning of one pass runs while the main stream
        #    still holds the features of the pass before it.
        main = torch.cuda.current_stream()
        side = self._side_stream(main.device)
        inputs_ready = torch.cuda.Event()
        inputs_ready.record(main)
        side.wait_event(inputs_ready)
        with torch.cuda.stream(side):
            # -- planning phase: everything whose size depends on the data, so that all
            #    host reads happen here and the feature phase is queued without waiting
            point._ensure_grid_coord()
            if "sparse_shape" in point.keys() and "_shape_pad" not in point.keys():
                # a caller's shape is the largest grid coordinate + 96 (sparsify's default pad,
                # model.py:162-164); the shapes of the coarse levels then follow without reading the device
                point["_shape_pad"] = 96
            if "sparse_shape" not in point.keys() or depth is None or "_counts" not in point.keys():
                stats = torch.cat([point.grid_coord.max(0).values.to(torch.int64), point.offset.to(torch.int64)])
                stats = stats.tolist()                                     # one host read
                if depth is None:
                    depth = max(stats[:3]).bit_length()
                if "sparse_shape" not in point.keys():
                    point["sparse_shape"] = [v + 96 for v in stats[:3]]
                    point["_shape_pad"] = 96
                off = [0] + stats[3:]
                point["_counts"] = [off[i + 1] - off[i] for i in range(len(off) - 1)]
            point.serialization(order=self.order, depth=depth, shuffle_orders=self.shuffle_orders)
            point["_sparse_indices"] = point._sparse_indices()
        # what was made there is consumed (and later dropped) by work queued on the main stream
        _record_stream(point, main)
        serialized = torch.cuda.Event()
        serialized.record(side)
        # the finest level's 3x3x3 kernel map is first needed after the stem: build it on the
        # second stream while the stem (which probes its own voxel index) runs on the first
        with torch.cuda.stream(side):
            kmaps0 = spconv.prebuild_kernel_map(
                point["_sparse_indices"], point.serialized_order[0], 3, status,
                with_pairs=_stage_uses_pairs(self.enc._modules.get("enc0"), point.batch.shape[0], feat_dtype))
        _record_stream(kmaps0, main)
        point["_prebuilt_kmaps"] = kmaps0
        events = {0: torch.cuda.Event()}
        events[0].record(side)
        stages = list(self.enc._modules.values())
        plan_state = {"cursor": point, "next": 0}

        def plan_upto(last):
            """Plans the pooling at the head of stages[next .. last] on the planning stream."""
            while plan_state["next"] <= min(last, len(stages) - 1):
                i = plan_state["next"]
                plan_state["next"] += 1
                stage, level = stages[i], plan_state["cursor"]
                down = stage[0] if len(stage) > 0 and isinstance(stage[0], SerializedPooling) else None
                if down is None:
                    if i == 0:
                        continue            # the finest stage has no pooling
                    plan_state["next"] = len(stages)
                    return
                with torch.cuda.stream(side):
                    child = down.plan(level)
                    level["_pooled_child"] = child
                    # the coarse level's 3x3x3 kernel map (and pair list where the pair-list
                    # convolution will be taken) only needs its coordinates: make it here too
                    child["_sparse_indices"] = child._sparse_indices()
                    child["_prebuilt_kmaps"] = spconv.prebuild_kernel_map(
                        child["_sparse_indices"], child.serialized_order[0], 3, status,
                        with_pairs=_stage_uses_pairs(stage, child.batch.shape[0], feat_dtype))
                    # ... and the patch layout of the stage's attention blocks
                    for m in stage:
                        if isinstance(m, Block) and m.attn.enable_flash:
                            m.attn.get_padding_and_inverse(child)
                            break
                # Everything made here was allocated on the planning stream but is consumed
                # (and some of it dropped) by work queued on the main stream: tell the
                # allocator, or a block freed after its last main-stream use was *queued*
                # could be handed to a later plan while that use has not run yet.
                _record_stream(child, main)
                events[i] = torch.cuda.Event()
                events[i].record(side)
                plan_state["cursor"] = child

        main.wait_event(serialized)
        point.sparsify()
        point = self.embedding(point)
        for i, stage in enumerate(stages):
            if i in events:
                main.wait_event(events[i])
            mods = list(stage._modules.values())
            if i == 0 and len(mods) > 1 and all(isinstance(m, Block) for m in mods):
                # the stem is one short kernel: queue the first block behind it before the
                # host turns to the first plan
                point = mods[0](point)
                plan_upto(1)
                for m in mods[1:]:
                    point = m(point)
            else:
                if i == 0:
                    plan_upto(1)
                point = stage(point)
            plan_upto(i + self.plan_ahead)
        if not self.cls_mode:
            point = self.dec(point)
        point["_defer_status"] = False
        if not self.defer_status_check:
            _lib.raise_on_status(status, "PointTransformerV3.forward")
        return point


class SegHead(PointModule):
    """Per-point classifier on the backbone's output: ``Linear(in_channels,
    num_classes)`` (state_dict keys ``weight`` / ``bias`` like the ``seg_head`` of a
    segmentor around the reference backbone) with the arg max taken in the same pass.
    ``forward(point)`` stores ``seg_logits`` (unless ``logits=False``) and ``seg_pred``."""

    def __init__(self, in_channels, num_classes, logits=True):
        super().__init__()
        self.linear = nn.Linear(in_channels, num_classes)
        self.logits = logits

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        # accept the flat keys of a plain nn.Linear head
        for k in ("weight", "bias"):
            if prefix + k in state_dict and prefix + "linear." + k not in state_dict:
                state_dict[prefix + "linear." + k] = state_dict.pop(prefix + k)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def forward(self, point):
        feat = point.feat if isinstance(point, Point) else point
        logits, labels = ops.seg_head(feat, self.linear.weight, self.linear.bias, want_logits=self.logits)
        if not isinstance(point, Point):
            return logits, labels
        if logits is not None:
            point["seg_logits"] = logits
        point["seg_pred"] = labels
        return point


def _linear_op(x, linear, status):
    """``linear(x)`` for an nn.Linear: on the tensor-core Linear kernels of the library where
    one takes the shape (bf16), else torch's own (fp32, unusual widths)."""
    if (type(linear) is nn.Linear and x.dtype == torch.bfloat16 and linear.weight.dtype == torch.bfloat16
            and x.dim() == 2):
        k, n_out = linear.in_features, linear.out_features
        if ops.gemm_supported(k, n_out, x.dtype):
            return ops.gemm(x, linear.weight, linear.bias, None, False, status)
        if linear.bias is not None and ops.linear_supported(k, n_out, False, x.dtype):
            return ops.linear(x, linear.weight, linear.bias, status)
    return linear(x)


def _stage_uses_pairs(stage, n, dtype):
    """Whether the 3x3x3 convolutions of the stage's blocks will ask for the pair list of this level
    (it is then made ahead of time with the kernel map; otherwise a convolution that wants one
    builds it when it runs)."""
    for m in (stage or []):
        if isinstance(m, Block):
            conv = m.cpe[0]
            return spconv.uses_pair_path(n, conv.in_channels, conv.out_channels, dtype, conv.kernel_size)
    return False


def _single_call_ok(feat, linear):
    """Whether a stage transition can go through its one-call entry point: bf16 features and
    parameters, a bias, a projection one of the tensor-core Linear kernels takes, no
    per-operator timing."""
    return (ops.TIMERS is None and feat.dtype == torch.bfloat16 and type(linear) is nn.Linear
            and linear.bias is not None and linear.weight.dtype == torch.bfloat16
            and linear.weight.is_contiguous()
            and ops.pool_stage_supported(linear.in_features, linear.out_features, feat.dtype))


def _record_stream(obj, stream):
    """tensor.record_stream(stream) for every CUDA tensor reachable through dicts,
    lists and tuples of ``obj``."""
    if isinstance(obj, torch.Tensor):
        if obj.is_cuda:
            obj.record_stream(stream)
    elif isinstance(obj, dict):
        for v in obj.values():
            _record_stream(v, stream)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            _record_stream(v, stream)


GridPooling = SerializedPooling
GridUnpooling = SerializedUnpooling
