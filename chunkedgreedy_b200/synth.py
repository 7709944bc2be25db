"""Seeded synthetic CSR generators for the five benchmark workloads.

The reference measures on SuiteSparse matrices that are not redistributable with
this repository; these generators stand in for them with the shapes, sizes and
value distributions of the named workloads.  Every generator returns
``(ptr, ind, val)`` as numpy arrays (int32, int32, float32): a square CSR matrix
with sorted, duplicate-free column indices, which is the input contract of the
reference library (sporder/include/sporder.h:26-27).

All randomness comes from ``numpy.random.default_rng(seed)`` so that the same
matrix is produced on every machine.
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "coo_to_csr",
    "zipf_banded",
    "stencil9",
    "road_lattice",
    "rmat",
    "rmat_gcn",
    "band",
    "random_sparse",
    "make_workload",
    "WORKLOADS",
]


def coo_to_csr(n, rows, cols, vals=None):
    """Sorted, duplicate-free CSR from COO (first value of a duplicate wins)."""
    key = np.asarray(rows).astype(np.int64)
    key *= np.int64(n)
    key += np.asarray(cols)
    if vals is None:
        key.sort()
        keep = np.empty(key.size, dtype=bool)
        keep[:1] = True
        np.not_equal(key[1:], key[:-1], out=keep[1:])
        key = key[keep]
        v = None
    else:
        key, first = np.unique(key, return_index=True)
        v = np.asarray(vals, dtype=np.float32)[first]
    r = key // n
    ind = (key - r * n).astype(np.int32)
    ptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(r, minlength=n), out=ptr[1:])
    return ptr.astype(np.int32), ind, v


def zipf_banded(n=65536, seed=0):
    """Workload 1: row length clip(3*Zipf(2),1,4096); 70 % of the columns within
    +-512 of a per-row centre, 30 % uniform; values U[-1,1]; rows permuted."""
    rng = np.random.default_rng(seed)
    length = np.clip(3 * rng.zipf(2.0, n), 1, 4096).astype(np.int64)
    centre = rng.integers(0, n, n)
    rows = np.repeat(np.arange(n, dtype=np.int64), length)
    total = int(length.sum())
    u = rng.random(total)
    near = (centre[rows] + rng.integers(-512, 513, total)) % n
    far = rng.integers(0, n, total)
    cols = np.where(u < 0.7, near, far)
    vals = rng.uniform(-1.0, 1.0, total).astype(np.float32)
    perm = rng.permutation(n)
    inv = np.empty(n, dtype=np.int64)
    inv[perm] = np.arange(n)
    return coo_to_csr(n, inv[rows], cols, vals)


def stencil9(side=1024, seed=1, relabel=True):
    """Workload 2: 9-point stencil on a side x side grid, symmetric N(0,1) values,
    rows and columns relabelled by one seeded permutation."""
    rng = np.random.default_rng(seed)
    n = side * side
    y, x = np.divmod(np.arange(n, dtype=np.int64), side)
    rr, cc = [], []
    for dy in (-1, 0, 1):
        for dx in (-1, 0, 1):
            ok = (y + dy >= 0) & (y + dy < side) & (x + dx >= 0) & (x + dx < side)
            rr.append(np.nonzero(ok)[0])
            cc.append((y[ok] + dy) * side + (x[ok] + dx))
    rows = np.concatenate(rr)
    cols = np.concatenate(cc)
    lo = np.minimum(rows, cols)
    hi = np.maximum(rows, cols)
    # one N(0,1) value per undirected edge, shared by (i,j) and (j,i)
    ukey, inverse = np.unique(lo * n + hi, return_inverse=True)
    vals = rng.standard_normal(ukey.size).astype(np.float32)[inverse]
    if relabel:
        q = rng.permutation(n)
        rows, cols = q[rows], q[cols]
    return coo_to_csr(n, rows, cols, vals)


def road_lattice(n=2_000_000, seed=2, relabel=True):
    """Workload 3: vertices on a jittered 2-D lattice, each linked to its 1-4
    nearest neighbours among the 8 surrounding lattice cells, symmetrised,
    unit weights, vertex ids relabelled."""
    rng = np.random.default_rng(seed)
    side = int(np.ceil(np.sqrt(n)))
    v = np.arange(n, dtype=np.int64)
    gy, gx = np.divmod(v, side)
    px = gx + rng.uniform(-0.5, 0.5, n)
    py = gy + rng.uniform(-0.5, 0.5, n)
    deg = rng.integers(1, 5, n)
    dist = np.full((n, 8), np.inf)
    nbr = np.zeros((n, 8), dtype=np.int64)
    j = 0
    for dy in (-1, 0, 1):
        for dx in (-1, 0, 1):
            if dy == 0 and dx == 0:
                continue
            ny, nx = gy + dy, gx + dx
            w = ny * side + nx
            ok = (ny >= 0) & (ny < side) & (nx >= 0) & (nx < side) & (w < n)
            wq = np.where(ok, w, 0)
            d = (px - px[wq]) ** 2 + (py - py[wq]) ** 2
            dist[:, j] = np.where(ok, d, np.inf)
            nbr[:, j] = wq
            j += 1
    order = np.argsort(dist, axis=1, kind="stable")
    rr, cc = [], []
    for t in range(4):
        pick = order[:, t]
        ok = (deg > t) & np.isfinite(dist[v, pick])
        rr.append(v[ok])
        cc.append(nbr[v[ok], pick[ok]])
    rows = np.concatenate(rr)
    cols = np.concatenate(cc)
    rows, cols = np.concatenate([rows, cols]), np.concatenate([cols, rows])
    if relabel:
        q = rng.permutation(n)
        rows, cols = q[rows], q[cols]
    ptr, ind, _ = coo_to_csr(n, rows, cols)
    return ptr, ind, np.ones(ind.size, dtype=np.float32)


def _rmat_edges(scale, edge_factor, probs, rng):
    a, b, c, _ = probs
    m = edge_factor << scale
    rows = np.zeros(m, dtype=np.int32)
    cols = np.zeros(m, dtype=np.int32)
    ab, abc, a32 = np.float32(a + b), np.float32(a + b + c), np.float32(a)
    for _level in range(scale):
        u = rng.random(m, dtype=np.float32)
        rbit = u >= ab  # quadrants c, d: row bit set
        cbit = u >= abc  # quadrant d ...
        cbit |= (u >= a32) & ~rbit  # ... or quadrant b: column bit set
        np.left_shift(rows, 1, out=rows)
        np.left_shift(cols, 1, out=cols)
        rows |= rbit
        cols |= cbit
    return rows, cols


def rmat(scale=22, edge_factor=16, probs=(0.57, 0.19, 0.19, 0.05), seed=3):
    """Workload 4: R-MAT, duplicates removed, values U(0,1]."""
    rng = np.random.default_rng(seed)
    n = 1 << scale
    rows, cols = _rmat_edges(scale, edge_factor, probs, rng)
    ptr, ind, _ = coo_to_csr(n, rows, cols)
    val = (1.0 - rng.random(ind.size, dtype=np.float32)).astype(np.float32)
    return ptr, ind, val


def rmat_gcn(scale=20, edge_factor=16, probs=(0.57, 0.19, 0.19, 0.05), seed=4):
    """Workload 5: R-MAT pattern symmetrised with self loops, values
    d_i^-1/2 d_j^-1/2 (the normalised GCN adjacency)."""
    rng = np.random.default_rng(seed)
    n = 1 << scale
    rows, cols = _rmat_edges(scale, edge_factor, probs, rng)
    loop = np.arange(n, dtype=np.int64)
    r = np.concatenate([rows, cols, loop])
    c = np.concatenate([cols, rows, loop])
    ptr, ind, _ = coo_to_csr(n, r, c)
    deg = np.diff(ptr).astype(np.float64)
    dis = 1.0 / np.sqrt(np.maximum(deg, 1.0))
    rr = np.repeat(np.arange(n), np.diff(ptr))
    val = (dis[rr] * dis[ind]).astype(np.float32)
    return ptr, ind, val


def band(n=1000, half=2):
    """Symmetric band pattern: row i holds columns i-half..i+half inside [0,n)
    (the fixture of the reference's C smoke test, sporder/tests/smoke.c:56-70)."""
    i = np.arange(n, dtype=np.int64)
    rr, cc = [], []
    for d in range(-half, half + 1):
        ok = (i + d >= 0) & (i + d < n)
        rr.append(i[ok])
        cc.append(i[ok] + d)
    ptr, ind, _ = coo_to_csr(n, np.concatenate(rr), np.concatenate(cc))
    return ptr, ind, np.ones(ind.size, dtype=np.float32)


def random_sparse(n, avg_deg, seed, symmetric=False, hub_cols=0, hub_frac=0.0,
                  empty_rows=0.0):
    """Small random pattern for parity tests; optional hub columns force the
    sketch into its eviction regime, optional empty rows exercise ragged input."""
    rng = np.random.default_rng(seed)
    m = int(n * avg_deg)
    rows = rng.integers(0, n, m)
    cols = rng.integers(0, n, m)
    if hub_cols > 0 and hub_frac > 0:
        h = int(m * hub_frac)
        hr = rng.integers(0, n, h)
        hc = rng.integers(0, hub_cols, h)
        rows = np.concatenate([rows, hr])
        cols = np.concatenate([cols, hc])
    if empty_rows > 0:
        dead = rng.random(n) < empty_rows
        keep = ~dead[rows]
        rows, cols = rows[keep], cols[keep]
        if symmetric:
            keep = ~dead[cols]
            rows, cols = rows[keep], cols[keep]
    if symmetric:
        rows, cols = np.concatenate([rows, cols]), np.concatenate([cols, rows])
    ptr, ind, _ = coo_to_csr(n, rows, cols)
    val = rng.uniform(-1.0, 1.0, ind.size).astype(np.float32)
    return ptr, ind, val


def dense_block(n, row0, rows, cols, seed, ragged=0, noise_deg=0.0):
    """``rows`` consecutive rows starting at ``row0`` that all hold columns ``[0, cols)``:
    every such row streams ``cols * (rows - 1)`` candidates, enough for the heavy-row path
    of the sketch stage at a few hundred rows.  With ``ragged`` > 0 row i stops
    ``i % ragged`` columns short (unequal Dice terms); otherwise all terms are equal, so
    weights tie all the time.  ``noise_deg`` adds random entries over the whole matrix."""
    rng = np.random.default_rng(seed)
    rr, cc = [], []
    for i in range(rows):
        c = cols - (i % ragged if ragged > 0 else 0)
        rr.append(np.full(c, row0 + i, dtype=np.int64))
        cc.append(np.arange(c, dtype=np.int64))
    if noise_deg > 0:
        m = int(n * noise_deg)
        rr.append(rng.integers(0, n, m))
        cc.append(rng.integers(0, n, m))
    ptr, ind, _ = coo_to_csr(n, np.concatenate(rr), np.concatenate(cc))
    val = rng.uniform(-1.0, 1.0, ind.size).astype(np.float32)
    return ptr, ind, val


def rotate_labels(ptr, ind, val, shift):
    """The same pattern with row and column r renamed (r + shift) mod n: moves the hub rows of
    an R-MAT matrix away from chunk 0."""
    n = ptr.size - 1
    rows = np.repeat(np.arange(n, dtype=np.int64), np.diff(ptr))
    ptr2, ind2, order = coo_to_csr(n, (rows + shift) % n, (ind.astype(np.int64) + shift) % n)
    return ptr2, ind2, val


WORKLOADS = {
    # name: (generator, kwargs, is_symmetric, dense widths for SpMM)
    "zipf65k": (zipf_banded, dict(n=65536, seed=0), False, (32,)),
    "stencil1024": (stencil9, dict(side=1024, seed=1), True, (32, 128)),
    # the same stencil in its natural (row-major grid) order: an input whose gathers hit the cache
    "stencil1024nat": (stencil9, dict(side=1024, seed=1, relabel=False), True, (32, 128)),
    "road2m": (road_lattice, dict(n=2_000_000, seed=2), True, (64,)),
    "rmat22": (rmat, dict(scale=22, edge_factor=16, seed=3), False, (32, 128, 256)),
    "rmat20gcn": (rmat_gcn, dict(scale=20, edge_factor=16, seed=4), True, (128, 16)),
}


def make_workload(name, **override):
    """Build a named workload; keyword overrides shrink it for tests
    (e.g. ``make_workload('rmat22', scale=14)``)."""
    gen, kwargs, sym, widths = WORKLOADS[name]
    kw = dict(kwargs)
    kw.update(override)
    ptr, ind, val = gen(**kw)
    return dict(name=name, ptr=ptr, ind=ind, val=val, is_symmetric=sym, widths=widths,
                n=int(ptr.size - 1), nnz=int(ind.size))
