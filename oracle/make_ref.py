"""Places the reference's own hot-path modules under oracle/_ref/ (git-ignored, never
committed) so that the CPU arm of bench.py can time the UNMODIFIED reference code.

    python oracle/make_ref.py [path-of-the-reference-checkout]

The source location is the argument, else the environment variable COMPLEXITY_DEEP_REFERENCE.
Only the pure-PyTorch packages the path needs are taken (complexity_deep/__init__.py, core/,
models/); the Triton package complexity_deep/cuda is not on the path and is left out.  The
files are copied byte for byte; nothing is patched.  TEST / BENCH INFRASTRUCTURE: nothing in
complexity_deep_b200 imports oracle/_ref.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make_ref(source: str | None = None) -> str | None:
    """Returns the destination directory, or None when no reference checkout is available."""
    source = source or os.environ.get("COMPLEXITY_DEEP_REFERENCE")
    if not source:
        return None
    pkg = os.path.join(source, "complexity_deep")
    if not os.path.isfile(os.path.join(pkg, "__init__.py")):
        return None
    out = os.path.join(DEST, "complexity_deep")
    if os.path.isdir(out):
        shutil.rmtree(out)
    os.makedirs(out)
    shutil.copy2(os.path.join(pkg, "__init__.py"), out)
    for sub in ("core", "models"):
        shutil.copytree(os.path.join(pkg, sub), os.path.join(out, sub),
                        ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return DEST


if __name__ == "__main__":
    dest = make_ref(sys.argv[1] if len(sys.argv) > 1 else None)
    print(dest if dest else "no reference checkout given (argument or COMPLEXITY_DEEP_REFERENCE)")
