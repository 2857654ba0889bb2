"""Copy the reference's Python package into ``oracle/_ref/`` so that it can travel with a snapshot of this tree.

    python oracle/make_ref.py [path to the reference checkout]        (default: $SEMICAT_REFERENCE, else DEFAULT_SRC)

The reference (olsdavis/semicat) is pure Python and has no ``setup.py`` / ``pyproject.toml``, so it cannot be
pip-installed; what the tests need from it is the package directory ``semicat/`` (the DiT in ``semicat/net/duo.py``,
the autograd glue in ``semicat/jvp_utils/functional.py`` and the Triton kernels beside it).  This script copies that
directory, unmodified, to ``oracle/_ref/semicat``.  ``oracle/_ref/`` is listed in ``.gitignore``: the copy is test
infrastructure on the machine that runs the tests, never part of this repository's history, and nothing in the
product imports it.  Only ``tests/`` and the comparator leg of ``bench.py`` do, through :func:`oracle.reference_root`.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_SRC = os.environ.get("SEMICAT_REFERENCE", "/root/reference")


def make(src_root: str = DEFAULT_SRC, force: bool = False) -> str | None:
    """Returns the destination directory, or None when the reference checkout is not available."""
    src = os.path.join(src_root, "semicat")
    if not os.path.isdir(src):
        return DEST if os.path.isdir(os.path.join(DEST, "semicat")) else None
    dst = os.path.join(DEST, "semicat")
    if os.path.isdir(dst):
        if not force:
            return DEST
        shutil.rmtree(dst)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as f:
        f.write(f"unmodified copy of {src} made by oracle/make_ref.py; not tracked by git\n")
    return DEST


if __name__ == "__main__":
    out = make(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SRC, force=True)
    print(out if out else "reference checkout not found; nothing copied")
