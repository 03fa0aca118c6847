"""The integer arithmetic of the CUDA encode kernel (magic-number bit spreading,
register Hilbert transform, compile-time Hilbert state-machine tables) compiled
for the host and compared with the oracle."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from oracle import cenc


@pytest.fixture(scope="module")
def hostlib(tmp_path_factory):
    so = str(tmp_path_factory.mktemp("hostmath") / "libencode_host.so")
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-o", so,
                           os.path.join(ROOT, "tests", "hostmath", "encode_host.cpp")])
    lib = ctypes.CDLL(so)
    lib.host_encode.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                ctypes.c_void_p]
    lib.host_decode.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return lib


@pytest.mark.parametrize("use_lut", [0, 1])
def test_kernel_integer_math_matches_oracle(hostlib, use_lut):
    rng = np.random.default_rng(5)
    for depth in range(1, 17):
        g = rng.integers(-3, (1 << depth) + 3, size=(4000, 3)).astype(np.int32)
        for oid, name in enumerate(["z", "z-trans", "hilbert", "hilbert-trans"]):
            out = np.empty(4000, dtype=np.int64)
            hostlib.host_encode(g.ctypes.data, 4000, depth, oid, use_lut, out.ctypes.data)
            assert (out == cenc.encode(g, None, depth, name)).all(), (depth, name)


def test_kernel_decode_math_inverts_encode(hostlib):
    rng = np.random.default_rng(6)
    for depth in range(1, 17):
        g = rng.integers(0, 1 << depth, size=(3000, 3)).astype(np.int64)
        for hilbert, name in ((0, "z"), (1, "hilbert")):
            code = cenc.encode(g, None, depth, name)
            out = np.empty((3000, 3), dtype=np.int64)
            hostlib.host_decode(code.ctypes.data, 3000, depth, hilbert, out.ctypes.data)
            assert (out == g).all(), (depth, name)
            assert (cenc.decode(code, depth, name)[0] == g).all()
