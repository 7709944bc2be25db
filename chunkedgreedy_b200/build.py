"""Build step of the CUDA library: nvcc, sm_100a only, in-tree output.

    python -m chunkedgreedy_b200.build [--force] [--verbose]

Produces chunkedgreedy_b200/libsporder_b200.so next to this file.  nvcc
cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libsporder_b200.so")
LIB_CHECKED = os.path.join(HERE, "libsporder_b200_checked.so")
SOURCES = ["api.cu", "transpose.cu", "sketch.cu", "greedy.cu", "reorder.cu", "spmm.cu", "pillars.cu"]
# No fast-math: the Dice terms need the IEEE fp32 divide and plain fp32 adds.
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "sporder_b200.h"))
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False, profile_rounds=False, checked=False):
    """``profile_rounds``: compile the chain kernel of the sketch stage with cycle counters per
    phase of a round (-DCSG_ROUND_PROFILE; a diagnostic build, slower, never the default).
    ``checked``: a second library, libsporder_b200_checked.so, in which every index a kernel
    derives from data of another kernel is tested before use (-DSPORDER_CHECKED); load it by
    setting SPORDER_B200_LIBRARY to its path."""
    if checked:
        return _build(LIB_CHECKED, "build_checked", ["-DSPORDER_CHECKED"], verbose)
    if not force and not profile_rounds and not needs_build():
        return LIB
    extra = ["-DCSG_ROUND_PROFILE=%d" % int(profile_rounds)] if profile_rounds else []
    return _build(LIB, "build", extra, verbose)


def _build(lib, objdir, extra, verbose):
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, objdir), exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(HERE, objdir, src.replace(".cu", ".o"))
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + extra + \
              ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                            text=True)))
        objs.append(obj)
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write("---- %s ----\n%s\n" % (src, out))
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([_nvcc(), "-shared", "-o", lib] + objs + ["-lcudart"])
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                profile_rounds=2 if "--profile-rounds=2" in sys.argv else int("--profile-rounds" in sys.argv),
                checked="--checked" in sys.argv))
