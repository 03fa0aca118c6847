"""The kernel-map entry point that uses the library's static device table
instead of a caller workspace (for hosts that cannot allocate device memory at
call time).  It must give exactly what the workspace-based entry point gives,
also on a second call that finds the previous call's entries in the table.

Collected last on purpose: a failure here must not hide any other test."""
import pytest
import torch

from helpers import small_batch
from pointtransformerv3_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _indices(sizes, seed):
    data = small_batch(sizes, seed)
    off = [0] + data["offset"].tolist()
    batch = torch.cat([torch.full((off[i + 1] - off[i],), i, dtype=torch.int32) for i in range(len(sizes))])
    return torch.cat([batch[:, None], data["grid_coord"].int()], 1).contiguous().cuda()


def _static_kmap(ind, ksize):
    """Calls ptv3_kmap_build_static through the C ABI; only outputs are allocated here."""
    lib = _lib.load()
    n = ind.shape[0]
    nbr = torch.full((ksize ** 3, n), -7, dtype=torch.int32, device=ind.device)
    status = torch.zeros(1, dtype=torch.int32, device=ind.device)
    rc = lib.ptv3_kmap_build_static(ind.data_ptr(), n, ksize, nbr.data_ptr(), status.data_ptr(),
                                    _lib.stream())
    return rc, nbr, int(status.item())


def test_static_kmap_equals_workspace_kmap_twice_in_a_row():
    lib = _lib.load()
    assert lib.ptv3_kmap_static_max_voxels() == 65536
    # two different clouds back to back: the second call must not see the first one's voxels
    for sizes, seed, ksize in (([5000, 3000], 71, 3), ([2000], 72, 5), ([5000, 3000], 71, 3)):
        ind = _indices(sizes, seed)
        rc, got, status = _static_kmap(ind, ksize)
        assert rc == 0, lib.ptv3_last_error()
        assert status == 0
        want = ops.kmap_build(ind, ksize)
        assert torch.equal(got, want)


def test_static_kmap_full_table_then_small_cloud_and_7x7x7():
    """The largest input the table serves (every slot range in use), a small cloud right after
    it (which finds the large one's entries beyond its own slots), and the 7x7x7 map."""
    lib = _lib.load()
    n = lib.ptv3_kmap_static_max_voxels()
    g = torch.Generator().manual_seed(5)
    # n distinct voxels of a 64 x 64 x 32 block in random row order, two scenes
    cells = torch.randperm(64 * 64 * 32, generator=g)[:n]
    ind = torch.stack([(torch.arange(n) >= n // 2).long(), cells // (64 * 32), (cells // 32) % 64, cells % 32],
                      1).int().contiguous().cuda()
    for cloud, ksize in ((ind, 3), (_indices([1500], 73), 3), (_indices([2500, 800], 74), 7), (ind, 5)):
        rc, got, status = _static_kmap(cloud, ksize)
        assert rc == 0, lib.ptv3_last_error()
        assert status == 0
        assert torch.equal(got, ops.kmap_build(cloud, ksize))


def test_static_kmap_rejects_inputs_beyond_its_table():
    lib = _lib.load()
    n = lib.ptv3_kmap_static_max_voxels() + 1
    ind = torch.zeros((n, 4), dtype=torch.int32, device="cuda")
    rc, _, _ = _static_kmap(ind, 3)
    assert rc == -2
    assert b"limit" in lib.ptv3_last_error()
