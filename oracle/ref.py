"""ctypes front end of the reference's own CUDA library built by oracle/build_ref.sh
(oracle/_ref/libsporder_ref.so).  Needs a GPU.  TEST INFRASTRUCTURE ONLY: used by the
GPU parity tests, by tests/golden/make_golden.py and by bench.py's comparison leg.

The reference aborts the process on invalid arguments, so only call it with
arguments its own checks accept.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import REF_SO

_lib = None


class RefTiming(C.Structure):
    _fields_ = [("wall_ms", C.c_double), ("csr2csc_ms", C.c_float),
                ("similarity_ms", C.c_float), ("chunk_greedy_ms", C.c_float)]


def available():
    return os.path.exists(REF_SO)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(REF_SO)
        _lib.sporder_context_create.restype = C.c_void_p
    return _lib


_ctx = None


def _context():
    global _ctx
    if _ctx is None:
        _ctx = C.c_void_p(lib().sporder_context_create())
    return _ctx


def csg(ptr, ind, is_symmetric=False, k=0, oversampling=0.0, chunk_size=0, with_timing=False):
    """sporder_chunk_similarity_greedy of the reference (sporder/include/sporder.h:224-228)
    on int32 CUDA torch tensors; returns the order tensor [, timing dict]."""
    import torch
    n, nnz = ptr.numel() - 1, ind.numel()
    order = torch.empty(n, dtype=torch.int32, device=ptr.device)
    torch.cuda.synchronize()
    t = RefTiming()
    lib().sporder_chunk_similarity_greedy(
        _context(), C.c_int32(n), C.c_int32(nnz), C.c_void_p(ptr.data_ptr()),
        C.c_void_p(ind.data_ptr()), C.c_bool(bool(is_symmetric)), C.c_int32(k),
        C.c_float(oversampling), C.c_int32(chunk_size), C.c_void_p(order.data_ptr()),
        C.byref(t) if with_timing else None, None)
    if with_timing:
        return order, dict(wall_ms=t.wall_ms, csr2csc_ms=t.csr2csc_ms,
                           similarity_ms=t.similarity_ms, chunk_greedy_ms=t.chunk_greedy_ms)
    return order


def csg_table(ptr, ind, is_symmetric, k, oversampling, chunk_size):
    """The reference's internal top-k table through oracle/ref_shim.cu; k, oversampling and
    chunk_size must be resolved values (the shim bypasses the C bridge's defaults)."""
    import torch
    n, nnz = ptr.numel() - 1, ind.numel()
    table = torch.empty((n, k), dtype=torch.int64, device=ptr.device)
    torch.cuda.synchronize()
    lib().refshim_csg_table(C.c_int32(n), C.c_int32(nnz), C.c_void_p(ptr.data_ptr()),
                            C.c_void_p(ind.data_ptr()), C.c_bool(bool(is_symmetric)),
                            C.c_int32(k), C.c_float(oversampling), C.c_int32(chunk_size),
                            C.c_void_p(table.data_ptr()))
    return table


def reorder(ptr, ind, new_order, val=None, symmetric=False):
    """sporder_reorder of the reference (sporder/include/sporder.h:253-258)."""
    import torch
    n, nnz = ptr.numel() - 1, ind.numel()
    ptr_new = torch.empty(n + 1, dtype=torch.int32, device=ptr.device)
    ind_new = torch.empty(max(nnz, 1), dtype=torch.int32, device=ptr.device)[:nnz]
    val_new = torch.empty(max(nnz, 1), dtype=torch.float32, device=ptr.device)[:nnz] \
        if val is not None else None
    torch.cuda.synchronize()
    lib().sporder_reorder(
        _context(), C.c_int32(n), C.c_int32(nnz), C.c_void_p(ptr.data_ptr()),
        C.c_void_p(ind.data_ptr()), C.c_void_p(val.data_ptr()) if val is not None else None,
        C.c_void_p(new_order.data_ptr()), C.c_int(1 if symmetric else 0),
        C.c_void_p(ptr_new.data_ptr()), C.c_void_p(ind_new.data_ptr()),
        C.c_void_p(val_new.data_ptr()) if val is not None else None)
    return (ptr_new, ind_new) if val is None else (ptr_new, ind_new, val_new)


def count_pillars(ptr, ind, height):
    """sporder_count_pillars of the reference (sporder/include/sporder.h:276-279) on int32
    CUDA torch tensors."""
    import torch
    n, nnz = ptr.numel() - 1, ind.numel()
    out = C.c_int32(0)
    torch.cuda.synchronize()
    lib().sporder_count_pillars(_context(), C.c_int32(n), C.c_int32(nnz), C.c_void_p(ptr.data_ptr()),
                                C.c_void_p(ind.data_ptr()), C.c_int32(int(height)), C.byref(out))
    return int(out.value)


def similarity_graph(ptr, ind, is_symmetric=False, k=0, oversampling=0.0):
    """sporder_similarity_graph of the reference (sporder/include/sporder.h:330-335) on int32
    CUDA torch tensors; returns (indices, weights) tensors of shape (n, k)."""
    import torch
    n, nnz = ptr.numel() - 1, ind.numel()
    kk = int(k) if k > 0 else min(32, max(16, 2 * (nnz // n)))
    idx = torch.empty((n, kk), dtype=torch.int32, device=ptr.device)
    wgt = torch.empty((n, kk), dtype=torch.float32, device=ptr.device)
    torch.cuda.synchronize()
    lib().sporder_similarity_graph(
        _context(), C.c_int32(n), C.c_int32(nnz), C.c_void_p(ptr.data_ptr()),
        C.c_void_p(ind.data_ptr()), C.c_bool(bool(is_symmetric)), C.c_int32(kk),
        C.c_float(oversampling), C.c_void_p(idx.data_ptr()), C.c_void_p(wgt.data_ptr()), None, None)
    torch.cuda.synchronize()
    return idx, wgt


def chunk_greedy(ptr, ind, is_symmetric=False, k=0, oversampling=0.0, chunk_size=0):
    """sporder_chunk_greedy of the reference (sporder/include/sporder.h:176-182) on int32
    CUDA torch tensors; returns the order tensor."""
    import torch
    n, nnz = ptr.numel() - 1, ind.numel()
    order = torch.empty(n, dtype=torch.int32, device=ptr.device)
    torch.cuda.synchronize()
    lib().sporder_chunk_greedy(
        _context(), C.c_int32(n), C.c_int32(nnz), C.c_void_p(ptr.data_ptr()),
        C.c_void_p(ind.data_ptr()), C.c_bool(bool(is_symmetric)), C.c_int32(k),
        C.c_float(oversampling), C.c_int32(chunk_size), C.c_void_p(order.data_ptr()), None, None)
    torch.cuda.synchronize()
    return order


def cusparse_spmm(ptr, ind, cols, warmup=3, repeat=10, seed=7):
    """sporder_bench_cusparse_spmm of the reference (sporder/include/sporder.h:295-299;
    sporder/src/bench_cusparse_spmm.cu:64-90): cusparseSpMM(CSR_ALG1) on the pattern with
    random fp32 values and a column-major dense operand of ``cols`` columns; returns the
    average milliseconds per launch."""
    import torch
    n, nnz = ptr.numel() - 1, ind.numel()
    ms = C.c_float(0.0)
    torch.cuda.synchronize()
    lib().sporder_bench_cusparse_spmm(
        _context(), C.c_int32(n), C.c_int32(nnz), C.c_void_p(ptr.data_ptr()),
        C.c_void_p(ind.data_ptr()), C.c_int32(int(cols)), C.c_int32(int(warmup)),
        C.c_int32(int(repeat)), C.c_uint64(int(seed)), C.byref(ms))
    torch.cuda.synchronize()
    return float(ms.value)
