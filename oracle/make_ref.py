"""Places the reference's own Python files under ``oracle/_ref/reference`` so that
the CPU arm of the benchmark can run the unmodified reference on a machine where
the reference checkout itself is absent.  TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [reference_root]

Copies ``model.py`` and ``serialization/*.py`` byte for byte (nothing is edited);
``oracle/_ref/`` is ignored by git, so the files never enter this repository's
history.  Without a reference checkout the script does nothing and returns 1.
The third-party packages that ``model.py`` imports are provided at run time by
the stand-ins in ``oracle/refshim`` (see ``oracle/refload.py``)."""
import glob
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = ("model.py", "LICENSE")


def make_ref(root=None):
    root = root or os.environ.get("PTV3_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(HERE)), "reference")
    if not os.path.isfile(os.path.join(root, "model.py")):
        return None
    dst = os.path.join(HERE, "_ref", "reference")
    os.makedirs(os.path.join(dst, "serialization"), exist_ok=True)
    for name in FILES:
        if os.path.isfile(os.path.join(root, name)):
            shutil.copyfile(os.path.join(root, name), os.path.join(dst, name))
    for src in glob.glob(os.path.join(root, "serialization", "*.py")):
        shutil.copyfile(src, os.path.join(dst, "serialization", os.path.basename(src)))
    return dst


if __name__ == "__main__":
    out = make_ref(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out or "no reference checkout found")
    sys.exit(0 if out else 1)
