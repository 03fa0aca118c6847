"""Thin tensor-level wrappers over the C ABI (one function per entry point).

Every wrapper allocates outputs and workspaces with torch, passes raw device
pointers and the current CUDA stream, and raises on a non-zero status."""
import ctypes

import torch

from . import _lib

ORDER_IDS = {"z": 0, "z-trans": 1, "hilbert": 2, "hilbert-trans": 3}


def encode(grid_coord, batch, depth, orders):
    """grid_coord (N,3) integer CUDA tensor, batch (N,) or None, orders: list of
    names -> (len(orders), N) int64 codes."""
    _lib.require_cuda(grid_coord, batch)
    lib = _lib.load()
    if grid_coord.dim() != 2 or grid_coord.shape[1] != 3:
        raise ValueError("grid_coord must be (N, 3), got %s" % (tuple(grid_coord.shape),))
    g = grid_coord.to(torch.int32).contiguous()
    n = g.shape[0]
    b = None
    if batch is not None:
        b = batch.to(torch.int64).contiguous()
        if b.shape != (n,):
            raise ValueError("batch must be (N,)")
    ids = (ctypes.c_int * len(orders))(*[ORDER_IDS[o] for o in orders])
    codes = torch.empty((len(orders), n), dtype=torch.int64, device=g.device)
    _lib.check(lib.ptv3_encode(_lib.ptr(g), _lib.ptr(b), n, int(depth), ids, len(orders),
                               _lib.ptr(codes), _lib.stream()), "ptv3_encode")
    return codes


def argsort_inverse(codes, sig_bits):
    """codes (k,N) int64 -> (order, inverse), both (k,N) int64, stable."""
    _lib.require_cuda(codes)
    lib = _lib.load()
    codes = codes.contiguous()
    k, n = codes.shape
    order = torch.empty_like(codes)
    inverse = torch.empty_like(codes)
    nbytes = lib.ptv3_argsort_workspace_bytes(k, n, int(sig_bits))
    ws = _lib.workspace(nbytes, codes.device)
    _lib.check(lib.ptv3_argsort_inverse(_lib.ptr(codes), k, n, int(sig_bits), _lib.ptr(order),
                                        _lib.ptr(inverse), _lib.ptr(ws), nbytes, _lib.stream()),
               "ptv3_argsort_inverse")
    return order, inverse
