"""Serialization codes with the reference's call signatures
(serialization/default.py:8-59), computed by the CUDA library."""
import torch

from .. import ops

_ORDERS = ("z", "z-trans", "hilbert", "hilbert-trans")


@torch.inference_mode()
def encode(grid_coord, batch=None, depth=16, order="z"):
    """(N,3) integer grid coordinates -> (N,) int64 codes, the scene id in the
    bits above 3*depth (serialization/default.py:8-24)."""
    assert order in _ORDERS
    return ops.encode(grid_coord, batch, depth, [order])[0]


def z_order_encode(grid_coord, depth=16):
    return ops.encode(grid_coord, None, depth, ["z"])[0]


def hilbert_encode(grid_coord, depth=16):
    return ops.encode(grid_coord, None, depth, ["hilbert"])[0]


@torch.inference_mode()
def decode(code, depth=16, order="z"):
    """Inverse of ``encode`` for the orders "z" and "hilbert"
    (serialization/default.py:27-38) -> (grid_coord (N,3) int64, batch (N,))."""
    assert order in {"z", "hilbert"}
    return ops.decode(code, depth, order)


def z_order_decode(code, depth=16):
    return ops.decode(code, depth, "z")[0]


def hilbert_decode(code, depth=16):
    return ops.decode(code, depth, "hilbert")[0]
