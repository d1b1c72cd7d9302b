"""Stage the reference package for runs on a box that does not have it.  TEST INFRASTRUCTURE ONLY.

    python oracle/stage_reference.py [path of the reference checkout]

The reference is a Python package that has to be imported under a package name
from its parent directory.  This recipe copies its harness modules (not its
docs, kernels or tools) from the checkout into ``oracle/_ref/moe_bench/`` - a
directory that is never committed - so that the GPU tests can drive this
library through the reference's OWN ``run_sweep`` / ``_time_run`` /
``verify_output`` (bench.py:52-153, reference.py:207-250) and its own input
generator, and so that the reference arm of the benchmark can time the
reference's own ``reference_moe``.  Nothing the library ships imports it.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "moe_bench")
MODULES = ("__init__.py", "baseline.py", "bench.py", "config.py", "context.py", "data.py", "distributed.py",
           "reference.py", "report.py", "schemes.py")


def default_source() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def stage(source: str | None = None) -> str | None:
    """Copy the harness modules; returns the staged package directory, or None when
    the checkout is not present (the previously staged copy, if any, is kept)."""
    source = source or default_source()
    if not os.path.isfile(os.path.join(source, "reference.py")):
        return DEST if os.path.isfile(os.path.join(DEST, "reference.py")) else None
    os.makedirs(DEST, exist_ok=True)
    for name in MODULES:
        shutil.copyfile(os.path.join(source, name), os.path.join(DEST, name))
    cfg_src = os.path.join(source, "configs")
    if os.path.isdir(cfg_src):
        shutil.copytree(cfg_src, os.path.join(DEST, "configs"), dirs_exist_ok=True)
    return DEST


def staged_parent() -> str | None:
    """Directory to put on ``sys.path`` so that ``import moe_bench`` finds the staged copy."""
    return os.path.dirname(DEST) if os.path.isfile(os.path.join(DEST, "reference.py")) else None


if __name__ == "__main__":
    path = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(path or "reference checkout not found; nothing staged")
