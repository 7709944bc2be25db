"""ctypes front end of the CPU checker (oracle/csg_oracle.c) and of the reference's
own CUDA build (oracle/_ref/libsporder_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke`` and by
the CPU-baseline legs of ``bench.py``; the product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from .build import ORACLE_SO, REF_SO, build_oracle

_lib = None


class CsgStats(C.Structure):
    _fields_ = [("k_used", C.c_int32), ("m_used", C.c_int32), ("avg_degree", C.c_double),
                ("avg_edge_weight", C.c_double), ("zero_degree_rows", C.c_int32),
                ("chunk_size_used", C.c_int32), ("chain_restarts", C.c_int32),
                ("avg_followed_weight", C.c_double)]

    def as_dict(self):
        return {f: getattr(self, f) for f, _ in self._fields_}


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build_oracle()
        _lib = C.CDLL(ORACLE_SO)
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def set_num_threads(t):
    lib().oracle_set_num_threads(C.c_int(int(t)))


def num_threads():
    return int(lib().oracle_num_threads())


def resolve_params(n, nnz, k=0, oversampling=0.0, chunk_size=0):
    """-> dict(k, oversampling, chunk_size, m_used, M) or raises ValueError."""
    kk, ov, ch = C.c_int32(k), C.c_float(oversampling), C.c_int32(chunk_size)
    mu, M = C.c_int32(0), C.c_int32(0)
    rc = lib().oracle_resolve_params(C.c_int32(n), C.c_int32(nnz), C.byref(kk), C.byref(ov),
                                     C.byref(ch), C.byref(mu), C.byref(M))
    if rc:
        raise ValueError("reference would abort: invalid k/oversampling (code %d)" % rc)
    return dict(k=kk.value, oversampling=ov.value, chunk_size=ch.value, m_used=mu.value, M=M.value)


def csg_table(ptr, ind, is_symmetric=False, k=0, oversampling=0.0, chunk_size=0):
    ptr, ind = _i32(ptr), _i32(ind)
    n, nnz = ptr.size - 1, ind.size
    prm = resolve_params(n, nnz, k, oversampling, chunk_size)
    table = np.zeros((n, prm["k"]), dtype=np.uint64)
    rc = lib().oracle_csg_table(C.c_int32(n), C.c_int32(nnz), _p(ptr), _p(ind),
                                C.c_int(bool(is_symmetric)), C.c_int32(prm["k"]),
                                C.c_float(prm["oversampling"]), C.c_int32(prm["chunk_size"]),
                                _p(table))
    if rc:
        raise ValueError("oracle_csg_table failed (%d)" % rc)
    return table


def greedy(table, n, chunk_size):
    table = np.ascontiguousarray(table, dtype=np.uint64)
    k = table.shape[1]
    order = np.empty(n, dtype=np.int32)
    r, l, w = C.c_int64(0), C.c_int64(0), C.c_double(0)
    lib().oracle_greedy(C.c_int32(n), C.c_int32(k), C.c_int32(chunk_size), _p(table), _p(order),
                        C.byref(r), C.byref(l), C.byref(w))
    return order, dict(restarts=r.value, links=l.value, link_weight_sum=w.value)


def csg(ptr, ind, is_symmetric=False, k=0, oversampling=0.0, chunk_size=0, with_table=False,
        with_stats=False, ncols=None):
    """Full pipeline.  Returns order [, table] [, stats dict].  ``ncols`` > n runs a
    block of whole chunks cut out of a wider matrix (pass k explicitly then)."""
    ptr, ind = _i32(ptr), _i32(ind)
    n, nnz = ptr.size - 1, ind.size
    ncols = n if ncols is None else int(ncols)
    prm = resolve_params(n, nnz, k, oversampling, chunk_size)
    order = np.empty(n, dtype=np.int32)
    table = np.zeros((n, prm["k"]), dtype=np.uint64) if with_table else None
    st = CsgStats()
    rc = lib().oracle_csg_rect(C.c_int32(n), C.c_int32(ncols), C.c_int32(nnz), _p(ptr), _p(ind),
                          C.c_int(bool(is_symmetric)), C.c_int32(k), C.c_float(oversampling),
                          C.c_int32(chunk_size), _p(order), _p(table),
                          C.byref(st) if with_stats else None)
    if rc:
        raise ValueError("oracle_csg failed (%d)" % rc)
    out = (order,)
    if with_table:
        out += (table,)
    if with_stats:
        out += (st.as_dict(),)
    return out if len(out) > 1 else out[0]


def reorder(ptr, ind, new_order, val=None, symmetric=False):
    ptr, ind, new_order = _i32(ptr), _i32(ind), _i32(new_order)
    n, nnz = ptr.size - 1, ind.size
    v = None if val is None else np.ascontiguousarray(val, dtype=np.float32)
    ptr_new = np.empty(n + 1, dtype=np.int32)
    ind_new = np.empty(nnz, dtype=np.int32)
    val_new = None if v is None else np.empty(nnz, dtype=np.float32)
    lib().oracle_reorder(C.c_int32(n), C.c_int32(nnz), _p(ptr), _p(ind), _p(v), _p(new_order),
                         C.c_int(1 if symmetric else 0), _p(ptr_new), _p(ind_new), _p(val_new))
    return (ptr_new, ind_new) if v is None else (ptr_new, ind_new, val_new)


def spmm_f64(ptr, ind, val, B, with_abs=True):
    ptr, ind = _i32(ptr), _i32(ind)
    val = np.ascontiguousarray(val, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    n, w = ptr.size - 1, B.shape[1]
    Cm = np.empty((n, w), dtype=np.float64)
    Ca = np.empty((n, w), dtype=np.float64) if with_abs else None
    lib().oracle_spmm_f64(C.c_int32(n), C.c_int32(w), _p(ptr), _p(ind), _p(val), _p(B), _p(Cm),
                          _p(Ca))
    return (Cm, Ca) if with_abs else Cm


def spmm_f32(ptr, ind, val, B):
    ptr, ind = _i32(ptr), _i32(ind)
    val = np.ascontiguousarray(val, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    n, w = ptr.size - 1, B.shape[1]
    Cm = np.empty((n, w), dtype=np.float32)
    lib().oracle_spmm_f32(C.c_int32(n), C.c_int32(w), _p(ptr), _p(ind), _p(val), _p(B), _p(Cm))
    return Cm


def similarity_graph(ptr, ind, k=0, oversampling=0.0):
    """The global top-k graph (sporder/src/similarity_graph.cu:26-107): the csg sketch with
    the whole matrix as the one chunk (sporder/src/common/similarity_top_k.cu:10-51) and the
    defaults of sporder/src/sporder.cpp:75-80.  Returns (indices, weights), shape (n, k)."""
    ptr, ind = _i32(ptr), _i32(ind)
    n, nnz = ptr.size - 1, ind.size
    if k <= 0:
        k = min(32, max(16, 2 * (nnz // n)))
    if oversampling <= 0.0:
        oversampling = 2.0
    _, table = csg(ptr, ind, False, k=k, oversampling=oversampling, chunk_size=n, with_table=True)
    return decode_table(table.reshape(n, k))


def chunk_greedy(ptr, ind, k=0, oversampling=0.0, chunk_size=0):
    """The reference's cg (sporder/src/cg/chunk_greedy.cu:118-163): global top-k graph with
    the defaults of sporder/src/sporder.cpp:118-126, then greedy chains per chunk.  Returns
    (order, stats dict) with the fraction of table weight that crosses chunk boundaries."""
    ptr, ind = _i32(ptr), _i32(ind)
    n, nnz = ptr.size - 1, ind.size
    if k <= 0:
        k = min(256, max(16, nnz // n))
    if oversampling <= 0.0:
        oversampling = 4.0
    if chunk_size <= 0:
        chunk_size = 1024
    _, table = csg(ptr, ind, False, k=k, oversampling=oversampling, chunk_size=n, with_table=True)
    table = table.reshape(n, k)
    order, st = greedy(table, n, chunk_size)
    idx, w = decode_table(table)
    rows = np.arange(n)[:, None]
    inside = (idx >= 0) & (idx // chunk_size == rows // chunk_size)
    total = float(w[idx >= 0].astype(np.float64).sum())
    st["cut_weight_fraction"] = (1.0 - float(w[inside].astype(np.float64).sum()) / total) if total > 0 else 0.0
    st["k_used"] = k
    return order, st


def count_pillars(ptr, ind, height, ncols=None):
    """Distinct (row // height, column) pairs (sporder/src/count_pillars.cu:38-85)."""
    ptr, ind = _i32(ptr), _i32(ind)
    n = ptr.size - 1
    if ncols is None:
        ncols = max(n, int(ind.max()) + 1 if ind.size else 1)
    fn = lib().oracle_count_pillars
    fn.restype = C.c_int64
    out = fn(C.c_int32(n), C.c_int32(ncols), _p(ptr), _p(ind), C.c_int32(height))
    if out < 0:
        raise ValueError("oracle_count_pillars: bad arguments")
    return int(out)


def decode_table(table):
    """packed entries -> (index int32, weight float32) arrays of the same shape."""
    t = np.asarray(table, dtype=np.uint64)
    idx = (t & np.uint64(0xFFFFFFFF)).astype(np.int64) - 1
    w = (t >> np.uint64(32)).astype(np.uint32).view(np.float32)
    return idx.astype(np.int32), w.reshape(t.shape)
