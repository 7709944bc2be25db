"""Seeded parity cases shared by the CPU tests, the GPU tests and the script that
records golden outputs of the reference library (tests/golden/make_golden.py)."""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from chunkedgreedy_b200 import synth  # noqa: E402


def _case(gen, sym=False, **params):
    return dict(gen=gen, is_symmetric=sym, params=params)


# name -> generator thunk, symmetry promise, csg keyword parameters.
# Sizes are kept small: the reference outputs of every case are committed as fixtures.
CASES = {
    # the fixture of the reference's own C smoke test (sporder/tests/smoke.c:56-70)
    "band1000": _case(lambda: synth.band(1000), True),
    # one row, one entry; empty rows; a chunk tail shorter than the chunk
    "tiny1": _case(lambda: synth.random_sparse(1, 1, 11)),
    "ragged": _case(lambda: synth.random_sparse(1500, 3, 12, empty_rows=0.3), False,
                    chunk_size=512),
    "uniform": _case(lambda: synth.random_sparse(3000, 6, 1)),
    # hub columns push most rows past the sketch capacity (eviction regime)
    "hubsym": _case(lambda: synth.random_sparse(2000, 8, 2, symmetric=True, hub_cols=40,
                                                hub_frac=0.5), True),
    "hub_c700": _case(lambda: synth.random_sparse(3000, 5, 3, hub_cols=30, hub_frac=0.6,
                                                  empty_rows=0.1), False, chunk_size=700),
    # capacity 96 (k=24, oversampling 3.5 -> m=84), three cells per lane
    "m96": _case(lambda: synth.random_sparse(2000, 12, 4, hub_cols=50, hub_frac=0.4), False,
                 k=24, oversampling=3.5, chunk_size=512),
    # smallest and largest capacities, k above one warp
    "m32": _case(lambda: synth.random_sparse(1500, 10, 5, hub_cols=20, hub_frac=0.5), False,
                 k=8, oversampling=1.0, chunk_size=256),
    "m512": _case(lambda: synth.random_sparse(1200, 40, 6, hub_cols=64, hub_frac=0.5), False,
                  k=40, oversampling=12.8, chunk_size=1024),
    # chunk covering the whole matrix (global similarity) and a 1-row chunk
    "onechunk": _case(lambda: synth.random_sparse(1800, 6, 7, hub_cols=25, hub_frac=0.4), False,
                      chunk_size=4096),
    "chunk1": _case(lambda: synth.random_sparse(300, 4, 8), False, chunk_size=1),
    # scaled-down versions of the five benchmark workloads
    "zipf4k": _case(lambda: synth.zipf_banded(n=4096, seed=0)),
    "stencil48": _case(lambda: synth.stencil9(side=48, seed=1), True),
    "stencil48_natural": _case(lambda: synth.stencil9(side=48, seed=1, relabel=False), True),
    "road3k": _case(lambda: synth.road_lattice(n=3000, seed=2), True),
    "rmat12": _case(lambda: synth.rmat(scale=12, seed=3)),
    "rmat11gcn": _case(lambda: synth.rmat_gcn(scale=11, seed=4), True),
}

# larger cases checked against the oracle only (no committed fixture)
BIG_CASES = {
    "rmat16": _case(lambda: synth.rmat(scale=16, seed=3)),
    "zipf65k": _case(lambda: synth.zipf_banded(n=65536, seed=0)),
    "stencil256": _case(lambda: synth.stencil9(side=256, seed=1), True),
    "rmat14gcn": _case(lambda: synth.rmat_gcn(scale=14, seed=4), True),
    "bigchunk": _case(lambda: synth.rmat(scale=13, seed=9), False, chunk_size=3000),
    # rows streaming more than 65536 candidates (the heavy-row path of the sketch stage):
    # equal Dice terms (weights tie all the time), fewer candidates than slots (the sketch
    # never fills), one cell per lane, unequal terms with noise, a 4096-row chunk, and a
    # chunk too large for the key tables (slots found by comparing keys)
    "dense_ties": _case(lambda: synth.dense_block(1024, 0, 300, 300, 21), False, k=16),
    "dense_fill": _case(lambda: synth.dense_block(2048, 10, 40, 2000, 22), False, k=16),
    "dense_m32": _case(lambda: synth.dense_block(1024, 0, 200, 400, 23), False, k=8,
                       oversampling=4.0),
    "dense_ragged": _case(lambda: synth.dense_block(2048, 100, 300, 320, 24, ragged=50,
                                                    noise_deg=3.0), False, k=16, chunk_size=512),
    "dense_c4096": _case(lambda: synth.dense_block(8192, 3000, 300, 300, 25, ragged=7), False,
                         k=16, chunk_size=4096),
    # three and four cells per lane on the heavy-row path
    "dense_m96": _case(lambda: synth.dense_block(1024, 0, 300, 300, 27, ragged=11), False, k=24,
                       oversampling=3.5),
    "dense_m128": _case(lambda: synth.dense_block(2048, 64, 320, 330, 28, ragged=40,
                                                  noise_deg=2.0), False, k=30),
    # eight cells per lane: beyond the sketches resolved in rounds (element-wise chain)
    "dense_m256": _case(lambda: synth.dense_block(1024, 0, 300, 300, 30, ragged=13), False, k=64),
    "dense_m128_ties": _case(lambda: synth.dense_block(1024, 0, 300, 300, 29), False, k=32),
    # hub rows in the middle of the matrix
    "rmat15_rotated": _case(lambda: synth.rotate_labels(*synth.rmat(scale=15, seed=5), 10240 + 77),
                            False, chunk_size=512),
    "dense_hugechunk": _case(lambda: synth.dense_block(60000, 50000, 280, 300, 26, ragged=3,
                                                       noise_deg=1.0), False, k=16,
                             chunk_size=60000),
}


def build(name):
    c = CASES.get(name) or BIG_CASES[name]
    ptr, ind, val = c["gen"]()
    return ptr, ind, val, c["is_symmetric"], dict(c["params"])
