"""The ``Point`` container of a batched point cloud with the reference's keys
and methods (model.py:28-174); serialization and kernel maps run on the CUDA
library."""
import torch

from . import _lib, ops
from .sparse import SparseConvTensor


@torch.inference_mode()
def offset2bincount(offset):
    """model.py:28-32."""
    return torch.diff(offset, prepend=torch.zeros(1, device=offset.device, dtype=torch.long))


@torch.inference_mode()
def offset2batch(offset, n=None):
    """model.py:35-40.  ``n``: the number of points when the caller knows it (the last
    offset); repeat_interleave then does not have to read its output size from the device."""
    bincount = offset2bincount(offset)
    ids = torch.arange(len(bincount), device=offset.device, dtype=torch.long)
    if n is None:
        return ids.repeat_interleave(bincount)
    return ids.repeat_interleave(bincount, output_size=int(n))


@torch.inference_mode()
def batch2offset(batch):
    """model.py:43-45."""
    return torch.cumsum(batch.bincount(), dim=0).long()


class AttrDict(dict):
    """Dictionary with attribute access whose constructor re-wraps nested
    dictionaries (the subset of ``addict.Dict`` the model relies on)."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        for a in args:
            if a is None:
                continue
            for k, v in (a.items() if isinstance(a, dict) else a):
                self[k] = self._wrap(v)
        for k, v in kwargs.items():
            self[k] = self._wrap(v)

    @classmethod
    def _wrap(cls, v):
        if type(v) is dict:
            return AttrDict(v)
        if isinstance(v, (list, tuple)) and not hasattr(v, "_fields"):
            return type(v)(cls._wrap(x) for x in v)
        return v

    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError:
            raise AttributeError(name) from None

    def __setattr__(self, name, value):
        self[name] = value

    def __delattr__(self, name):
        try:
            del self[name]
        except KeyError:
            raise AttributeError(name) from None


class Point(AttrDict):
    """Batched point cloud (model.py:48-79).  Keys: ``coord``, ``grid_coord``,
    ``offset``/``batch``, ``feat``, ``grid_size``; after ``serialization()``:
    ``serialized_depth/code/order/inverse``; after ``sparsify()``:
    ``sparse_shape``, ``sparse_conv_feat``.

    ``_counts`` (host list of per-scene point counts) is a cache this
    implementation adds so that sizes are known without further device reads."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        if "batch" not in self.keys() and "offset" in self.keys():
            n = None
            for k in ("feat", "grid_coord", "coord"):      # any per-point tensor tells the size
                if k in self.keys() and torch.is_tensor(self[k]):
                    n = self[k].shape[0]
                    break
            if n is not None and self.offset.is_cuda:
                self["batch"] = ops.batch_indices(self.offset, n)[0]      # one kernel of this library
            else:
                self["batch"] = offset2batch(self.offset, n)
        elif "offset" not in self.keys() and "batch" in self.keys():
            self["offset"] = batch2offset(self.batch)

    def device_status(self):
        """The device status word kernels OR error bits into (created on first use
        and shared with the levels pooled from this one)."""
        if "_status" not in self.keys():
            ref = self.feat if "feat" in self.keys() else self.batch
            self["_status"] = ops.new_status(ref.device)
        return self["_status"]

    def check_status(self, what="point operators", force=False):
        """Raises if a kernel reported a problem.  Reads the status word (a host
        sync) unless the owner of the forward pass deferred the check to its end."""
        if "_status" in self.keys() and (force or not self.get("_defer_status", False)):
            _lib.raise_on_status(self["_status"], what)

    def host_counts(self):
        """Per-scene point counts as Python ints (one device read, then cached)."""
        if "_counts" not in self.keys():
            off = [0] + self.offset.tolist()
            self["_counts"] = [off[i + 1] - off[i] for i in range(len(off) - 1)]
        return self["_counts"]

    def _ensure_grid_coord(self):
        if "grid_coord" not in self.keys():
            assert {"grid_size", "coord"}.issubset(self.keys())
            self["grid_coord"] = torch.div(
                self.coord - self.coord.min(0)[0], self.grid_size, rounding_mode="trunc").int()

    def serialization(self, order="z", depth=None, shuffle_orders=False):
        """model.py:81-136: codes of every requested order, their stable argsort
        and inverse; rows optionally shuffled with ``torch.randperm`` on the
        CPU generator exactly as the reference draws it."""
        assert "batch" in self.keys()
        self._ensure_grid_coord()
        order = [order] if isinstance(order, str) else list(order)
        if depth is None:
            depth = int(self.grid_coord.max()).bit_length()
        depth = max(int(depth), 1)
        self["serialized_depth"] = depth
        n_scene_bits = len(self.offset).bit_length()
        assert depth * 3 + n_scene_bits <= 63
        assert depth <= 16
        if shuffle_orders:
            # the reference shuffles the finished rows (model.py:128-132); the rows are independent of
            # each other, so the same draw applied to the list of orders gives the same tensors
            # without re-stacking them
            perm = torch.randperm(len(order)).tolist()
            order = [order[i] for i in perm]
        code = ops.encode(self.grid_coord, self.batch, depth, order)
        sorted_order, inverse = ops.argsort_inverse(code, depth * 3 + n_scene_bits, self.device_status())
        self.check_status("ptv3_argsort_inverse")
        self["serialized_code"] = code
        self["serialized_order"] = sorted_order
        self["serialized_inverse"] = inverse

    def _sparse_indices(self):
        """(N, 4) int32 rows (batch, x, y, z); a copy prepared together with the level's
        pooling plan is used when there is one."""
        ready = self.pop("_sparse_indices", None)
        if ready is not None:
            return ready
        if self.grid_coord.is_cuda and "offset" in self.keys():
            return ops.batch_indices(self.offset, self.grid_coord.shape[0], self.grid_coord, want_batch=False)[1]
        return torch.cat([self.batch.unsqueeze(-1).int(), self.grid_coord.int()], dim=1).contiguous()

    def sparsify(self, pad=96):
        """model.py:138-174: wraps the features and (batch, x, y, z) indices in a
        SparseConvTensor for the submanifold convolutions."""
        assert {"feat", "batch"}.issubset(self.keys())
        self._ensure_grid_coord()
        if "sparse_shape" in self.keys():
            sparse_shape = self.sparse_shape
        else:
            sparse_shape = torch.add(torch.max(self.grid_coord, dim=0).values, pad).tolist()
            self["_shape_pad"] = pad
        self["sparse_shape"] = sparse_shape
        self["sparse_conv_feat"] = SparseConvTensor(
            features=self.feat,
            indices=self._sparse_indices(),
            spatial_shape=sparse_shape,
            batch_size=len(self.offset),
            row_order=self.serialized_order[0] if "serialized_order" in self.keys() else None,
            status=self.device_status(),
            defer_status=self.get("_defer_status", False),
            prebuilt=self.pop("_prebuilt_kmaps", None),
        )
