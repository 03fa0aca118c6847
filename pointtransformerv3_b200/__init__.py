"""B200-native inference path of Point Transformer V3 behind the reference's API."""
from . import serialization
from .point import Point, batch2offset, offset2batch, offset2bincount
from .sparse import SparseConvTensor, SubMConv3d
from .voxelize import voxelize
from .model import (Block, Embedding, GridPooling, GridUnpooling, MLP, PDNorm, PointModule, PointSequential, RPE,
                    PointTransformerV3, SegHead, SerializedAttention, SerializedPooling, SerializedUnpooling)

__all__ = ["serialization", "Point", "batch2offset", "offset2batch", "offset2bincount", "SparseConvTensor",
           "SubMConv3d", "Block", "Embedding", "GridPooling", "GridUnpooling", "MLP", "PDNorm", "PointModule", "RPE",
           "PointSequential", "PointTransformerV3", "SerializedAttention", "SerializedPooling",
           "SerializedUnpooling", "SegHead", "voxelize"]
