"""Copy the reference's Python package next to this file, unmodified.

    REFERENCE_ROOT=<reference checkout> python baseline/fetch_reference.py

The reference ships its attention kernels as Triton source that is compiled when
first called, so "installing" it for a comparison on the GPU means having its
``lazy_attn/lazy`` package importable there.  This script copies that package
(Python files only, byte for byte) into ``baseline/_ref/lazy_attn/lazy``.  The
target directory is ignored by git: the copy exists only in a working tree, for
the GPU tests and the benchmark's Triton leg (``baseline/triton_ref.py``), and is
never part of this project's history.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref" / "lazy_attn" / "lazy"


def fetch(reference_root=None, quiet=False) -> bool:
    """Returns True when the copy exists afterwards."""
    root = reference_root or os.environ.get("REFERENCE_ROOT")
    if not root:
        return TARGET.exists()
    src = Path(root) / "lazy_attn" / "lazy"
    if not src.is_dir():
        if not quiet:
            print(f"no reference package at {src}", file=sys.stderr)
        return TARGET.exists()
    if TARGET.exists():
        shutil.rmtree(TARGET)
    shutil.copytree(src, TARGET, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    if not quiet:
        n = sum(1 for _ in TARGET.rglob("*.py"))
        print(f"copied {n} files to {TARGET}")
    return True


if __name__ == "__main__":
    raise SystemExit(0 if fetch() else 1)
