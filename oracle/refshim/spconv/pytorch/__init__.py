"""CPU stand-in for the parts of spconv.pytorch the reference model touches."""
import math

import torch
import torch.nn as nn

from oracle import ptv3_oracle as _o


class SparseConvTensor:
    def __init__(self, features, indices, spatial_shape, batch_size, indice_dict=None):
        self.features = features
        self.indices = indices
        self.spatial_shape = spatial_shape
        self.batch_size = batch_size
        self.indice_dict = {} if indice_dict is None else indice_dict

    def replace_feature(self, feature):
        return SparseConvTensor(feature, self.indices, self.spatial_shape, self.batch_size,
                                self.indice_dict)


class SparseModule(nn.Module):
    pass


class SubMConv3d(SparseModule):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1,
                 groups=1, bias=True, indice_key=None, **kw):
        super().__init__()
        k = kernel_size
        self.kernel_size = k
        self.indice_key = indice_key
        self.weight = nn.Parameter(torch.empty(out_channels, k, k, k, in_channels))
        nn.init.kaiming_uniform_(self.weight.view(out_channels, -1), a=math.sqrt(5))
        self.bias = nn.Parameter(torch.zeros(out_channels)) if bias else None

    def forward(self, x):
        key = (self.indice_key, self.kernel_size)
        if self.indice_key is None or key not in x.indice_dict:
            nbr = _o.kernel_map(x.indices, self.kernel_size)
            if self.indice_key is not None:
                x.indice_dict[key] = nbr
        else:
            nbr = x.indice_dict[key]
        return x.replace_feature(_o.subm_conv(x.features, nbr, self.weight, self.bias))


class _Modules:
    @staticmethod
    def is_spconv_module(m):
        return isinstance(m, SparseModule)


modules = _Modules()
