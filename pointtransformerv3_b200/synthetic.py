"""Seeded synthetic point clouds that stand in for the indoor scans and LiDAR
sweeps the reference is trained on (no dataset is available offline).  All
generators run on the CPU generator ``torch.Generator().manual_seed(seed)`` so
that the same seed gives the same cloud on every machine."""
import math

import torch


def _voxel_dedup(coord, grid_size):
    """Keeps the first point of every occupied voxel; returns (coord, grid_coord)."""
    gc = torch.div(coord - coord.min(0)[0], grid_size, rounding_mode="trunc").to(torch.int64)
    key = (gc[:, 0] << 42) | (gc[:, 1] << 21) | gc[:, 2]
    uniq, inv = torch.unique(key, return_inverse=True)
    first = torch.full((uniq.shape[0],), coord.shape[0], dtype=torch.int64)
    first.scatter_reduce_(0, inv, torch.arange(coord.shape[0]), "amin")
    first = torch.sort(first).values
    return coord[first], gc[first].int()


def uniform_cloud(n=100_000, extent=10.0, grid_size=0.02, seed=0):
    """Serialization-only workload: xyz uniform in [0, extent]^3, duplicates kept."""
    g = torch.Generator().manual_seed(seed)
    xyz = torch.rand(n, 3, generator=g) * extent
    gc = torch.div(xyz - xyz.min(0)[0], grid_size, rounding_mode="trunc").int()
    return xyz, gc


def indoor_scene(seed=0, target_voxels=100_000, grid_size=0.02, room=(10.0, 10.0, 3.0),
                 n_rect=20):
    """Points sampled on ``n_rect`` axis-aligned rectangles inside a room, then
    voxelised and de-duplicated.  The rectangle sides are scaled so that about
    ``target_voxels`` voxels are occupied."""
    g = torch.Generator().manual_seed(seed)
    room_t = torch.tensor(room)
    # total area needed ~ target * grid^2 ; sides U[1,2]*s  =>  mean area 2.25 s^2 (ignoring overlap)
    s = math.sqrt(target_voxels * grid_size ** 2 / (n_rect * 2.25)) * 1.02
    pts = []
    for i in range(n_rect):
        axis = i % 3
        a, b = [d for d in range(3) if d != axis]
        side = (1.0 + torch.rand(2, generator=g)) * s
        side = torch.minimum(side, room_t[[a, b]])
        lo = torch.rand(2, generator=g) * (room_t[[a, b]] - side)
        h = torch.rand(1, generator=g) * room_t[axis]
        n_raw = int(6 * side[0] * side[1] / grid_size ** 2)
        uv = torch.rand(n_raw, 2, generator=g) * side + lo
        p = torch.empty(n_raw, 3)
        p[:, a], p[:, b], p[:, axis] = uv[:, 0], uv[:, 1], h
        pts.append(p)
    coord = torch.cat(pts)
    coord = coord[torch.randperm(coord.shape[0], generator=g)]
    return _voxel_dedup(coord, grid_size)


def lidar_scene(seed=0, grid_size=0.05, n_sweeps=2, beams=64, azimuth_steps=2048, max_range=50.0):
    """A spinning-LiDAR-like sweep: ``beams`` elevations from -25 to +3 degrees,
    ``azimuth_steps`` azimuths, rays hit the ground plane or one of 10-30 random
    boxes; ``n_sweeps`` sweeps from sensor positions ~1 m apart are merged."""
    g = torch.Generator().manual_seed(seed)
    n_box = 10 + int(torch.randint(0, 21, (1,), generator=g))
    centre = (torch.rand(n_box, 2, generator=g) - 0.5) * 2 * 40.0
    half = 0.5 + torch.rand(n_box, 3, generator=g) * torch.tensor([3.0, 3.0, 2.5])
    lo = torch.cat([centre - half[:, :2], torch.zeros(n_box, 1)], 1)
    hi = torch.cat([centre + half[:, :2], 2 * half[:, 2:]], 1)
    elev = torch.deg2rad(torch.linspace(-25.0, 3.0, beams))
    azim = torch.arange(azimuth_steps) * (2 * math.pi / azimuth_steps)
    d = torch.stack([torch.cos(elev)[:, None] * torch.cos(azim)[None, :],
                     torch.cos(elev)[:, None] * torch.sin(azim)[None, :],
                     torch.sin(elev)[:, None].expand(-1, azimuth_steps)], -1).reshape(-1, 3)
    pts = []
    for s in range(n_sweeps):
        origin = torch.tensor([1.0 * s, 0.3 * s, 1.8])
        t = torch.full((d.shape[0],), float("inf"))
        down = d[:, 2] < -1e-6
        t[down] = -origin[2] / d[down, 2]
        inv = 1.0 / torch.where(d.abs() < 1e-9, torch.full_like(d, 1e-9), d)
        for b in range(n_box):
            t0 = (lo[b] - origin) * inv
            t1 = (hi[b] - origin) * inv
            tn = torch.minimum(t0, t1).max(1).values
            tf = torch.maximum(t0, t1).min(1).values
            hit = (tn <= tf) & (tn > 0)
            t = torch.where(hit & (tn < t), tn, t)
        ok = t < max_range
        noise = 1.0 + 0.002 * torch.randn(int(ok.sum()), generator=g)
        pts.append(origin + d[ok] * (t[ok] * noise)[:, None])
    coord = torch.cat(pts)
    return _voxel_dedup(coord, grid_size)


def make_batch(scenes, extra_channels, seed=0, dtype=torch.float32):
    """scenes: list of (coord, grid_coord).  feat = cat(coord, uniform[0,1) extras)."""
    g = torch.Generator().manual_seed(10_000 + seed)
    coord = torch.cat([s[0] for s in scenes])
    grid = torch.cat([s[1] for s in scenes])
    counts = torch.tensor([s[0].shape[0] for s in scenes], dtype=torch.int64)
    feat = torch.cat([coord, torch.rand(coord.shape[0], extra_channels, generator=g)], 1).to(dtype)
    return dict(coord=coord, grid_coord=grid, feat=feat, offset=torch.cumsum(counts, 0))


def indoor_batch(n_scenes=4, first_seed=0, target_voxels=100_000, grid_size=0.02, dtype=torch.float32):
    scenes = [indoor_scene(first_seed + i, target_voxels, grid_size) for i in range(n_scenes)]
    return make_batch(scenes, 3, first_seed, dtype)


def lidar_batch(n_scenes=16, first_seed=0, grid_size=0.05, dtype=torch.float32):
    scenes = [lidar_scene(first_seed + i, grid_size) for i in range(n_scenes)]
    return make_batch(scenes, 1, first_seed, dtype)
