"""Voxelisation front end: from raw points to the one-point-per-voxel batch the
backbone takes (the step before ``PointTransformerV3.forward``).

The reference derives ``grid_coord`` itself when it is missing (model.py:88-96)
but leaves the choice of one point per voxel to its data pipeline; here both run
on the GPU (``ptv3_grid_coord``, ``ptv3_voxel_dedup``)."""
import torch

from . import ops
from .point import offset2batch


@torch.inference_mode()
def voxelize(coord, feat, offset, grid_size, extra=None):
    """coord (N, 3) float, feat (N, C), offset (B,) cumulative counts, all on the GPU.

    Returns (data_dict, point2voxel): ``data_dict`` has ``coord``, ``grid_coord``,
    ``feat``, ``offset``, ``grid_size`` of the first point of every occupied voxel
    (scenes stay contiguous, rows stay in input order) and can be passed to the
    backbone; ``point2voxel`` (N,) maps every input point to its row there, for
    scattering per-voxel results back to points.  ``extra``: optional dict of
    further per-point tensors to carry along.  One host read (the voxel count)."""
    offset = offset.to(torch.int64)
    batch = offset2batch(offset, coord.shape[0])
    grid, _ = ops.grid_coord(coord, grid_size)
    indices = torch.cat([batch.unsqueeze(-1).int(), grid], dim=1).contiguous()
    d = ops.voxel_dedup(indices, offset)
    keep = d["keep"]
    out = {"coord": coord.index_select(0, keep), "grid_coord": grid.index_select(0, keep),
           "feat": feat.index_select(0, keep), "offset": d["offset"], "grid_size": grid_size}
    for k, v in (extra or {}).items():
        out[k] = v.index_select(0, keep)
    return out, d["point2voxel"]
