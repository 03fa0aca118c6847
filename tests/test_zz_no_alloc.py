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


def test_static_kmap_rejects_inputs_beyond_its_table():
    lib = _lib.load()
    n = lib.ptv3_kmap_static_max_voxels() + 1
    ind = torch.zeros((n, 4), dtype=torch.int32, device="cuda")
    rc, _, _ = _static_kmap(ind, 3)
    assert rc == -2
    assert b"limit" in lib.ptv3_last_error()
