"""Imports the unmodified reference (when its tree is present) for validation
and golden-vector generation.  TEST INFRASTRUCTURE ONLY; returns None where the
reference tree does not exist (e.g. on a GPU box)."""
import importlib
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root():
    """Directory of the reference's files: $PTV3_REFERENCE_ROOT, else a `reference`
    directory next to this repository, else the copy `oracle/make_ref.py` placed under
    `oracle/_ref/reference`."""
    if "PTV3_REFERENCE_ROOT" in os.environ:
        return os.environ["PTV3_REFERENCE_ROOT"]
    sibling = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if os.path.isfile(os.path.join(sibling, "model.py")):
        return sibling
    return os.path.join(_HERE, "_ref", "reference")


def load_serialization():
    root = reference_root()
    if not os.path.isdir(os.path.join(root, "serialization")):
        return None
    parent = os.path.dirname(root)
    if parent not in sys.path:
        sys.path.append(parent)
    return importlib.import_module(os.path.basename(root) + ".serialization")


def load_model():
    """The reference model module, imported through the stand-in packages."""
    root = reference_root()
    if not os.path.isfile(os.path.join(root, "model.py")):
        return None
    shim = os.path.join(_HERE, "refshim")
    repo = os.path.dirname(_HERE)
    for p in (shim, repo):
        if p not in sys.path:
            sys.path.insert(0, p)
    parent = os.path.dirname(root)
    if parent not in sys.path:
        sys.path.append(parent)
    return importlib.import_module(os.path.basename(root) + ".model")
