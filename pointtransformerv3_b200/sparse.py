"""The slice of spconv's interface the model uses (SparseConvTensor,
SubMConv3d, modules.is_spconv_module; call sites model.py:165-172, :233-249,
:546-552, :767-774), implemented on the CUDA library's kernel map and
submanifold convolution."""
import math

import torch
import torch.nn as nn

from . import ops


# The pair-list convolution multiplies only the (input, output) pairs that exist, 128 pairs of one
# offset at a time, so a slice of the weights serves 128 useful rows; an output-stationary tile of a
# coarse level uses it for the ~40 voxels of its 128 that have that neighbour.  That pays only when the
# weights are nearly all of the traffic.  Measured on the coarsest level of the default backbone
# (2 238 voxels, 512 channels): 0.083 ms on the pair list, 0.062 ms on the kernel map; so the
# default backbone never takes this path, and it starts at twice that width.
PAIR_PATH_MAX_VOXELS = 65536
PAIR_PATH_MIN_CHANNELS = 1024


def uses_pair_path(n, in_channels, out_channels, dtype, kernel_size=3):
    """Whether a 3x3x3 convolution of this shape runs on the pair list (else on the kernel map)."""
    return (dtype == torch.bfloat16 and kernel_size == 3 and n <= PAIR_PATH_MAX_VOXELS
            and in_channels >= PAIR_PATH_MIN_CHANNELS and in_channels % 64 == 0 and out_channels % 128 == 0)


class SparseConvTensor:
    """features (N,C), indices (N,4) int32 rows (batch, x, y, z).  Kernel maps
    are cached in ``indice_dict`` under ``(indice_key, kernel_size)`` and shared
    by every tensor derived with ``replace_feature``."""

    def __init__(self, features, indices, spatial_shape, batch_size, indice_dict=None, row_order=None,
                 status=None, defer_status=False, prebuilt=None):
        self.features = features
        self.indices = indices
        self.spatial_shape = spatial_shape
        self.batch_size = batch_size
        self.indice_dict = {} if indice_dict is None else indice_dict
        # optional voxel permutation along a space-filling curve; convolutions
        # group voxels into tiles in this order (an extension, not in spconv)
        self.row_order = row_order
        # device status word of the owning Point; when the check is deferred the
        # owner reads it once at the end of its forward pass
        self.status = status
        self.defer_status = defer_status
        # kernel maps / pair lists made ahead of time for this voxel set, by kernel size
        # (whatever indice_key a convolution names): {ksize: (nbr, row_order)}, {(ksize, "pairs"): ...}
        self.prebuilt = {} if prebuilt is None else prebuilt

    def replace_feature(self, feature):
        return SparseConvTensor(feature, self.indices, self.spatial_shape, self.batch_size, self.indice_dict,
                                self.row_order, self.status, self.defer_status, self.prebuilt)

    def kernel_map(self, kernel_size, indice_key=None):
        """(nbr, row_order): the offset-major neighbour table with its columns in
        ``row_order`` (natural order when that is None)."""
        key = (indice_key, kernel_size)
        if indice_key is not None and key in self.indice_dict:
            return self.indice_dict[key]
        if kernel_size in self.prebuilt:
            entry = self.prebuilt[kernel_size]
            if indice_key is not None:
                self.indice_dict[key] = entry
            return entry
        nbr = ops.kmap_build(self.indices, kernel_size, self.status, self.row_order)
        if self.status is not None and not self.defer_status:
            from . import _lib
            _lib.raise_on_status(self.status, "ptv3_kmap_build")
        entry = (nbr, self.row_order)
        if indice_key is not None:
            self.indice_dict[key] = entry
        return entry

    def pair_list(self, kernel_size, indice_key=None):
        """Offset-sorted pair list of the kernel map (built once per key)."""
        key = (indice_key, kernel_size, "pairs")
        if indice_key is not None and key in self.indice_dict:
            return self.indice_dict[key]
        if (kernel_size, "pairs") in self.prebuilt:
            pairs = self.prebuilt[(kernel_size, "pairs")]
            if indice_key is not None:
                self.indice_dict[key] = pairs
            return pairs
        nbr, row_order = self.kernel_map(kernel_size, indice_key)
        pairs = ops.conv_pairs_build(nbr, row_order)
        if indice_key is not None:
            self.indice_dict[key] = pairs
        return pairs


class SparseModule(nn.Module):
    """Marker base class (what ``is_spconv_module`` looks for)."""


class SubMConv3d(SparseModule):
    """Submanifold 3-D convolution: outputs only at the input's active voxels.
    ``weight`` is (out, k, k, k, in); ``padding``/``stride``/``dilation`` other
    than the defaults do not change a submanifold convolution's output sites
    and only unit stride/dilation are supported."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, indice_key=None, algo=None, fp32_accum=None, **unused):
        super().__init__()
        if not isinstance(kernel_size, int):
            assert len(set(kernel_size)) == 1, "only cubic kernels are supported"
            kernel_size = kernel_size[0]
        assert kernel_size % 2 == 1 and kernel_size <= 7
        assert stride in (1, (1, 1, 1), [1, 1, 1]) and dilation in (1, (1, 1, 1), [1, 1, 1]) and groups == 1
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = kernel_size
        self.indice_key = indice_key
        k = kernel_size
        self.weight = nn.Parameter(torch.empty(out_channels, k, k, k, in_channels))
        self.bias = nn.Parameter(torch.empty(out_channels)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        fan_in = self.in_channels * self.kernel_size ** 3
        bound = 1.0 / math.sqrt(fan_in)
        nn.init.uniform_(self.weight, -bound, bound)
        if self.bias is not None:
            nn.init.uniform_(self.bias, -bound, bound)

    def uses_direct_path(self):
        """Few input channels with a large kernel: probing the hash table inside
        the convolution beats building a (kernel volume x N) neighbour table."""
        return self.in_channels <= 8 and self.kernel_size == 5 and self.out_channels in (16, 32, 48, 64)

    def forward(self, x, bn_scale=None, bn_shift=None, gelu=False):
        if self.uses_direct_path():
            out = ops.subm_conv_direct(x.features, x.indices, self.weight, self.bias, bn_scale, bn_shift, gelu,
                                       x.row_order, x.status)
            if x.status is not None and not x.defer_status:
                from . import _lib
                _lib.raise_on_status(x.status, "ptv3_subm_conv_direct_fwd")
            return x.replace_feature(out)
        assert bn_scale is None and not gelu
        geo = self.geometry(x)
        if "pair_in" in geo:
            return x.replace_feature(ops.subm_conv_pairs(x.features, geo, self.weight, self.bias))
        out = ops.subm_conv(x.features, geo["nbr"], self.weight, self.bias, row_order=geo["row_order"],
                            status=x.status if x.defer_status else None)
        return x.replace_feature(out)

    def geometry(self, x):
        """The index structure this convolution runs on for the sparse tensor ``x``:
        the pair list on the coarsest levels (few voxels, very wide channels: only the
        pairs that exist are multiplied), else dict(nbr, row_order) of the kernel map."""
        if uses_pair_path(x.features.shape[0], self.in_channels, self.out_channels, x.features.dtype,
                          self.kernel_size):
            return x.pair_list(self.kernel_size, self.indice_key)
        nbr, row_order = x.kernel_map(self.kernel_size, self.indice_key)
        return {"nbr": nbr, "row_order": row_order}


class _Modules:
    @staticmethod
    def is_spconv_module(module):
        return isinstance(module, SparseModule)


modules = _Modules()


def prebuild_kernel_map(indices, row_order, kernel_size, status, with_pairs):
    """Kernel map (and optionally its pair list) of a voxel set, in the form
    SparseConvTensor(prebuilt=...) takes."""
    nbr = ops.kmap_build(indices, kernel_size, status, row_order)
    out = {kernel_size: (nbr, row_order)}
    if with_pairs:
        out[(kernel_size, "pairs")] = ops.conv_pairs_build(nbr, row_order)
    return out
