"""Shared helpers of the parity tests."""
import torch


def small_scene(n, seed, grid_size=0.02, extent=2.0):
    """A bumpy surface, voxelised and de-duplicated: (coord fp32, grid_coord int32)."""
    g = torch.Generator().manual_seed(seed)
    xy = torch.rand(n, 2, generator=g) * extent
    z = 0.3 * torch.sin(xy[:, 0] * 3) + 0.05 * torch.rand(n, generator=g)
    c = torch.cat([xy, z[:, None]], 1)
    gc = torch.div(c - c.min(0)[0], grid_size, rounding_mode="trunc").to(torch.int64)
    key = (gc[:, 0] << 40) | (gc[:, 1] << 20) | gc[:, 2]
    uniq, inv = torch.unique(key, return_inverse=True)
    first = torch.full((uniq.shape[0],), n, dtype=torch.int64)
    first.scatter_reduce_(0, inv, torch.arange(n), "amin")
    first = torch.sort(first).values
    return c[first], gc[first].int()


def small_batch(sizes, seed=0, extra=3):
    scenes = [small_scene(n, seed * 100 + i) for i, n in enumerate(sizes)]
    coord = torch.cat([s[0] for s in scenes])
    grid = torch.cat([s[1] for s in scenes])
    counts = torch.tensor([s[0].shape[0] for s in scenes], dtype=torch.int64)
    g = torch.Generator().manual_seed(seed + 999)
    feat = torch.cat([coord, torch.rand(coord.shape[0], extra, generator=g)], 1)
    return dict(coord=coord, grid_coord=grid, feat=feat, offset=torch.cumsum(counts, 0))


def assert_close(got, ref, atol, rtol, what=""):
    got, ref = got.float().cpu(), ref.float().cpu()
    err = (got - ref).abs()
    bound = atol + rtol * ref.abs()
    bad = err > bound
    assert not bool(bad.any()), "%s: %d/%d outside atol=%g rtol=%g, max err %g (ref max %g)" % (
        what, int(bad.sum()), bad.numel(), atol, rtol, float(err.max()), float(ref.abs().max()))


def assert_close_chain(got, ref, atol, rtol, what="", frac=1e-3, factor=2.0):
    """For the output of a CHAIN of bf16 operators.  The one-operator tolerance must hold for
    all but `frac` of the elements, and `factor` times that tolerance for every element.
    Where the oracle and a kernel round an intermediate value to different bf16 neighbours,
    the following LayerNorm / GEMM / residual sum carries that ulp on, and after a residual
    sum that cancels (large operands, small result) one ulp of an operand exceeds a bound
    taken relative to the result; the strict form cannot hold for every element then."""
    g, r = got.float().cpu(), ref.float().cpu()
    err = (g - r).abs()
    outside = err > atol + rtol * r.abs()
    share = float(outside.float().mean())
    assert share <= frac, "%s: %.3g of the elements outside atol=%g rtol=%g" % (what, share, atol, rtol)
    assert_close(got, ref, factor * atol, factor * rtol, what)


def rel_l2(got, ref):
    got, ref = got.float().cpu(), ref.float().cpu()
    return float((got - ref).norm() / ref.norm().clamp_min(1e-30))


# tolerances of the feature path: bf16 max-abs 2e-2 / rel 1e-2, fp32 1e-4
TOL = {torch.float32: dict(atol=1e-4, rtol=1e-4), torch.bfloat16: dict(atol=2e-2, rtol=1e-2)}
