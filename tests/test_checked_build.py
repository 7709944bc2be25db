"""The checked build of the library (-DSPORDER_CHECKED: every index a kernel derives from
data another kernel wrote is tested before use, the first violation is reported instead of
followed) on the parity cases: same results as the CPU restatement, and no violation."""
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import sys
import numpy as np
import torch
sys.path.insert(0, %(root)r)
sys.path.insert(0, %(tests)r)
import cases, oracle
import chunkedgreedy_b200 as sp
from chunkedgreedy_b200 import _lib
assert _lib.LIB_PATH.endswith("_checked.so"), _lib.LIB_PATH
names = list(cases.CASES) + ["dense_ties", "dense_fill", "dense_ragged", "dense_m96", "dense_m128",
                             "dense_c4096", "dense_m256", "dense_hugechunk", "rmat16", "bigchunk"]
for name in names:
    ptr, ind, val, sym, params = cases.build(name)
    dp, di, dv = (torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (ptr, ind, val))
    order, table = sp.csg_table(dp, di, is_symmetric=sym, **params)
    o, t = oracle.csg(ptr, ind, sym, with_table=True, **params)
    assert np.array_equal(table.cpu().numpy().view(np.uint64), t), name
    assert np.array_equal(order.cpu().numpy(), o), name
    p2, i2, v2 = sp.reorder(dp, di, order, val=dv, symmetric=True)
    rp, ri, rv = oracle.reorder(ptr, ind, o, val, symmetric=True)
    assert np.array_equal(i2.cpu().numpy(), ri) and np.array_equal(v2.cpu().numpy(), rv), name
    assert sp.count_pillars(dp, di, 16) == oracle.count_pillars(ptr, ind, 16), name
    # the route that runs one chunk ahead on a second stream, forced for every size
    ctxa = sp.Context()
    ctxa.set_ahead_threshold(1)
    for _ in range(2):
        o3, t3 = sp.csg_table(dp, di, is_symmetric=False, ctx=ctxa, **params)
        assert np.array_equal(t3.cpu().numpy().view(np.uint64), t) and np.array_equal(o3.cpu().numpy(), o), name
    ctxa.close()
    if not sym:  # a false promise of symmetry: garbage candidates, but every index in bounds
        o2 = sp.chunk_similarity_greedy(dp, di, is_symmetric=True, **params)
        assert np.array_equal(np.sort(o2.cpu().numpy()), np.arange(ptr.size - 1)), name
print("checked build: %%d cases clean" %% len(names))
"""


def test_checked_build_agrees_and_reports_nothing():
    from chunkedgreedy_b200 import build
    if not os.path.exists(build.LIB_CHECKED):
        pytest.skip("checked library not built (python -m chunkedgreedy_b200.build --checked)")
    env = dict(os.environ, SPORDER_B200_LIBRARY=build.LIB_CHECKED)
    script = SCRIPT % {"root": ROOT, "tests": os.path.join(ROOT, "tests")}
    out = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "cases clean" in out.stdout
