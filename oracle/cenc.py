"""ctypes access to the C restatement of the serialization stage (test oracle)."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libptv3_oracle.so")
ORDER_IDS = {"z": 0, "z-trans": 1, "hilbert": 2, "hilbert-trans": 3}


def build(force=False):
    src = os.path.join(_HERE, "encode_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        i64p = ctypes.POINTER(ctypes.c_int64)
        i32p = ctypes.POINTER(ctypes.c_int32)
        _lib.oracle_encode.argtypes = [i32p, i64p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, i64p]
        _lib.oracle_argsort_stable.argtypes = [i64p, ctypes.c_int64, i64p]
        _lib.oracle_inverse.argtypes = [i64p, ctypes.c_int64, i64p]
        _lib.oracle_decode.argtypes = [i64p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, i64p, i64p]
    return _lib


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def encode(grid_coord, batch, depth, order):
    """grid_coord (N,3) integer array, batch (N,) or None -> (N,) int64 codes."""
    g = np.ascontiguousarray(np.asarray(grid_coord), dtype=np.int32).reshape(-1, 3)
    n = g.shape[0]
    out = np.empty(n, dtype=np.int64)
    b = None if batch is None else np.ascontiguousarray(np.asarray(batch), dtype=np.int64)
    rc = lib().oracle_encode(_p(g, ctypes.c_int32), None if b is None else _p(b, ctypes.c_int64),
                             n, int(depth), ORDER_IDS[order], _p(out, ctypes.c_int64))
    if rc != 0:
        raise ValueError("oracle_encode rc=%d" % rc)
    return out


def argsort_stable(code):
    c = np.ascontiguousarray(code, dtype=np.int64)
    order = np.empty(c.shape[0], dtype=np.int64)
    rc = lib().oracle_argsort_stable(_p(c, ctypes.c_int64), c.shape[0], _p(order, ctypes.c_int64))
    if rc != 0:
        raise RuntimeError("oracle_argsort_stable rc=%d" % rc)
    return order


def inverse(order):
    o = np.ascontiguousarray(order, dtype=np.int64)
    inv = np.empty_like(o)
    rc = lib().oracle_inverse(_p(o, ctypes.c_int64), o.shape[0], _p(inv, ctypes.c_int64))
    if rc != 0:
        raise ValueError("oracle_inverse rc=%d" % rc)
    return inv


def decode(code, depth, order):
    """(N,) int64 codes -> (grid_coord (N,3) int64, batch (N,) int64); order "z" or "hilbert"."""
    c = np.ascontiguousarray(code, dtype=np.int64).reshape(-1)
    grid = np.empty((c.shape[0], 3), dtype=np.int64)
    batch = np.empty(c.shape[0], dtype=np.int64)
    rc = lib().oracle_decode(_p(c, ctypes.c_int64), c.shape[0], int(depth), ORDER_IDS[order],
                             _p(grid, ctypes.c_int64), _p(batch, ctypes.c_int64))
    if rc != 0:
        raise ValueError("oracle_decode rc=%d" % rc)
    return grid, batch
