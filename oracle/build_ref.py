"""Stages the reference's own CPU implementation of the path for timing (TEST INFRASTRUCTURE).

    python oracle/build_ref.py <reference checkout>

Copies the reference's numpy package (python/polarquant_kv) and its Lloyd-Max codebook module
(src/polarquant_kv_cuda/lloyd_max.py) unmodified into oracle/_ref/, which version control ignores:
the files never become part of this repository, they only sit beside it so that the CPU-baseline leg
of the benchmark can time the reference as shipped on whatever host runs it.  There is nothing to
compile: the reference's CPU path is pure Python.  Only the benchmark's CPU-baseline leg and the
tests may import oracle/_ref; the shipped package never does.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def stage(reference_root: str) -> str | None:
    pkg = os.path.join(reference_root, "python", "polarquant_kv")
    lm = os.path.join(reference_root, "src", "polarquant_kv_cuda", "lloyd_max.py")
    if not os.path.isdir(pkg) or not os.path.isfile(lm):
        return None
    os.makedirs(DEST, exist_ok=True)
    dst_pkg = os.path.join(DEST, "polarquant_kv")
    if os.path.isdir(dst_pkg):
        shutil.rmtree(dst_pkg)
    shutil.copytree(pkg, dst_pkg, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    shutil.copyfile(lm, os.path.join(DEST, "ref_lloyd_max.py"))
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    out = stage(sys.argv[1])
    print(out if out else f"no reference checkout at {sys.argv[1]}")
