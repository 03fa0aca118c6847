"""Scene-level data parallelism: every rank runs the backbone on its own group
of scenes; the only collective is the gather of the output features.

Scenes never interact inside the backbone (patches, clusters and kernel maps
are per scene, BatchNorm is in eval mode), so no exchange is needed during the
forward.  Two quantities are batch-global in the reference and must be made
global here: the serialization depth (Hilbert codes depend on it) and the CPU
random generator state that draws the order shuffles."""
import torch
import torch.distributed as dist


def shard_scenes(n_scenes, rank, world):
    """Contiguous scene range [lo, hi) of this rank."""
    per, rem = divmod(n_scenes, world)
    lo = rank * per + min(rank, rem)
    return lo, lo + per + (1 if rank < rem else 0)


def slice_batch(data, lo, hi):
    """Sub-batch with scenes [lo, hi) of a data dict (coord, grid_coord, feat, offset)."""
    off = [0] + data["offset"].tolist()
    a, b = off[lo], off[hi]
    out = {k: v[a:b] for k, v in data.items() if k != "offset" and torch.is_tensor(v) and v.dim() > 0
           and v.shape[0] == off[-1]}
    out["offset"] = data["offset"][lo:hi] - a
    return out


def global_depth(grid_coord, group=None):
    """Serialization depth over all ranks' coordinates (model.py:98-101 evaluated
    on the whole batch): one 8-byte all-reduce(max)."""
    m = grid_coord.max().to(torch.int64).reshape(1)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
    return max(int(m.item()).bit_length(), 1)


def gather_features(feat, group=None):
    """All-gathers per-rank feature matrices of different lengths.

    Returns (features of all ranks concatenated in rank order, list of row
    counts).  Rows are padded to the longest rank for one all_gather_into_tensor
    over NCCL; the padding is dropped afterwards."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return feat, [feat.shape[0]]
    world = dist.get_world_size(group)
    n = torch.tensor([feat.shape[0]], dtype=torch.int64, device=feat.device)
    counts = torch.empty(world, dtype=torch.int64, device=feat.device)
    dist.all_gather_into_tensor(counts, n, group=group)
    counts = counts.tolist()
    longest = max(counts)
    send = feat
    if feat.shape[0] != longest:
        send = torch.zeros((longest,) + tuple(feat.shape[1:]), dtype=feat.dtype, device=feat.device)
        send[: feat.shape[0]] = feat
    recv = torch.empty((world * longest,) + tuple(feat.shape[1:]), dtype=feat.dtype, device=feat.device)
    dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
    parts = [recv[r * longest: r * longest + counts[r]] for r in range(world)]
    return torch.cat(parts), counts
