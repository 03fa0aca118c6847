"""CPU-only checks of the boundary: the shared library builds, loads and
exports every symbol the public header declares (no compute call is made)."""
import ctypes
import os
import re

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ptv3_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ptv3_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from pointtransformerv3_b200 import _lib, build
    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 5
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header must list the same symbols"


def test_version_and_error_string():
    from pointtransformerv3_b200 import _lib
    lib = _lib.load()
    assert lib.ptv3_version() >= 1
    assert isinstance(lib.ptv3_last_error(), bytes)


def test_cpu_tensor_is_rejected_loudly():
    import pytest
    import torch
    from pointtransformerv3_b200 import _lib, ops
    with pytest.raises(_lib.Ptv3Error):
        ops.encode(torch.zeros(4, 3, dtype=torch.int32), None, 16, ["z"])
