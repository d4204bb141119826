"""Recipe that places an unmodified copy of the reference's Python package under ``oracle/_ref/``
(test / baseline infrastructure; the directory is git-ignored and never read by the product path).

The reference is pure Python, so "building" it is a file copy of its ``leankv`` package from the
checkout named by ``LEANKV_REFERENCE_DIR`` (default ``/root/reference``). Where no checkout is
present (the GPU box), a copy made earlier is used as it is. ``load()`` imports the copy under its
own name and redirects nothing: the reference writes its Lloyd-Max codebook cache next to its own
``codebook.py``, which here is the copy, not the checkout.
"""

from __future__ import annotations

import importlib
import os
import shutil
import sys

_DIR = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_DIR, "_ref")
PKG_DIR = os.path.join(REF_DIR, "leankv")


def build(force: bool = False) -> str | None:
    """Copy the reference package if a checkout is present. Returns the copy's path, or None when
    there is neither a checkout nor an earlier copy."""
    src = os.path.join(os.environ.get("LEANKV_REFERENCE_DIR", "/root/reference"), "leankv")
    if os.path.isdir(src) and (force or not os.path.isdir(PKG_DIR)):
        os.makedirs(REF_DIR, exist_ok=True)
        if os.path.isdir(PKG_DIR):
            shutil.rmtree(PKG_DIR)
        shutil.copytree(src, PKG_DIR, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return PKG_DIR if os.path.isdir(PKG_DIR) else None


def available() -> bool:
    return os.path.isfile(os.path.join(PKG_DIR, "__init__.py"))


def load():
    """Import the copied reference package (``import leankv``). Raises ImportError if it is absent."""
    if not available():
        raise ImportError("no copy of the reference package under oracle/_ref (run oracle/build_ref.py "
                          "where a reference checkout is present)")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module("leankv")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
