"""Build recipes for the checker: the C restatement (always) and the reference's
own CUDA library (only where the reference checkout is present).

    python -m oracle.build            # both
    python -m oracle.build --oracle   # C restatement only

Outputs: oracle/liboracle.so and oracle/_ref/libsporder_ref.so (both git-ignored).
Test infrastructure only; the product library never links or loads either.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libsporder_ref.so")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "csg_oracle.c")
    if force or _stale(ORACLE_SO, [src]):
        cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-ffp-contract=off",
               "-fno-fast-math", "-fvisibility=hidden", "-Wall", "-Wextra", "-o", ORACLE_SO,
               src, "-lm"]
        subprocess.check_call(cmd)
    return ORACLE_SO


def reference_root():
    """Where the reference checkout lies: SPORDER_REFERENCE_ROOT, else the sibling directory
    ``reference`` of this repository; None when neither holds the sporder sources."""
    here_parent = os.path.dirname(os.path.dirname(HERE))
    for cand in (os.environ.get("SPORDER_REFERENCE_ROOT"), os.path.join(here_parent, "reference")):
        if cand and os.path.isdir(os.path.join(cand, "sporder", "src")):
            return cand
    return None


def build_ref(ref_root=None, force=False):
    """Compile the unmodified reference sources in place (needs ~4 min, no GPU)."""
    ref_root = ref_root or reference_root()
    if not ref_root or not os.path.isdir(os.path.join(ref_root, "sporder", "src")):
        return REF_SO if os.path.exists(REF_SO) else None
    shim = os.path.join(HERE, "ref_shim.cu")
    if force or _stale(REF_SO, [shim, os.path.join(HERE, "build_ref.sh")]):
        subprocess.check_call(["bash", os.path.join(HERE, "build_ref.sh"), ref_root])
    return REF_SO


if __name__ == "__main__":
    build_oracle(force="--force" in sys.argv)
    if "--oracle" not in sys.argv:
        build_ref(force="--force" in sys.argv)
