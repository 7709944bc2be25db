"""B200-native Chunked Greedy (csg) reordering, permutation application and SpMM.

The compute entry points keep the keyword surface of the reference's Python
package (sporder/python/sporder/__init__.py:113-149 ``reorder`` and :380-424
``chunk_similarity_greedy``): same argument names and meaning, same return
shapes (a bare array, or a tuple with ``timing`` and/or ``stats`` appended when
requested), permutations in new2old form.  Use it as
``import chunkedgreedy_b200 as sporder``.

Arrays are CUDA tensors (``torch.Tensor``) or any object that exports DLPack /
``__cuda_array_interface__``; results come back in the framework of the first
array argument (torch tensors for torch input; ``<framework>.from_dlpack`` of the
result otherwise, as in sporder/python/sporder/__init__.py:28-39), on the same
device.  All work is done by hand-written sm_100a kernels behind the C ABI in
``include/sporder_b200.h``; there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C

from . import _lib

__all__ = ["Context", "chunk_similarity_greedy", "reorder", "spmm", "csg_table",
           "chunk_similarity_greedy_host", "kernel_launches", "count_pillars",
           "similarity_graph", "chunk_greedy"]

_default_ctx = {}


def _torch():
    import torch
    return torch


class Context:
    """Owns a CUDA stream and a device workspace, bound to the device current at
    creation, or to ``device`` when given (sporder/include/sporder.h:43-52).  One context
    per thread or device; a context serves one stream at a time (re-binding it to another
    stream first waits for the work it queued on the previous one)."""

    def __init__(self, device=None):
        torch = _torch()
        if not torch.cuda.is_available():
            raise RuntimeError("chunkedgreedy_b200 needs a CUDA device (no CPU fallback)")
        lib = _lib.load()
        torch.cuda.init()
        self.device = torch.cuda.current_device() if device is None else int(device)
        with torch.cuda.device(self.device):
            # make sure the primary context exists before the library asks for the device
            torch.empty(1, device="cuda")
            self._h = lib.sporder_context_create()
        if not self._h:
            _lib.check()
            raise RuntimeError("sporder_context_create failed")

    @property
    def handle(self):
        return self._h

    def workspace_bytes(self):
        return int(_lib.load().sporder_context_workspace_bytes(self._h))

    def set_stream_limit(self, max_elements):
        """Upper bound (stream elements of 8 bytes, 0 = none) on the buffer for the heaviest
        rows' materialised candidate streams; results never depend on it."""
        _lib.load().sporder_context_set_stream_limit(self._h, int(max_elements))

    def set_ahead_threshold(self, min_nnz):
        """Nonzeros from which a csg call runs its heaviest chunk ahead of the rest on a second
        stream: 0 = the built-in rule, > 0 = every call of at least that many nonzeros, < 0 =
        never.  Results never depend on it."""
        _lib.load().sporder_context_set_ahead_threshold(self._h, int(min_nnz))

    def close(self):
        if getattr(self, "_h", None):
            _lib.load().sporder_context_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _ctx(ctx, ref=None):
    """The caller's context, or the shared default context of the device the arrays live on
    (created on first use; sporder/python/bindings.cpp:40-43 keeps one such singleton)."""
    if ctx is not None:
        return ctx
    torch = _torch()
    dev = ref.device.index if ref is not None and ref.is_cuda else torch.cuda.current_device()
    if dev is None:
        dev = torch.cuda.current_device()
    if dev not in _default_ctx:
        _default_ctx[dev] = Context(device=dev)
    return _default_ctx[dev]


def _like(result, reference):
    """``result`` (a torch tensor) in the array framework ``reference`` came from
    (sporder/python/sporder/__init__.py:28-39): torch stays torch, any other framework that
    offers ``from_dlpack`` (CuPy, ...) receives a zero-copy view."""
    torch = _torch()
    if result is None or isinstance(reference, torch.Tensor):
        return result
    root = type(reference).__module__.partition(".")[0]
    if root in ("torch", "builtins", "numpy", ""):
        return result
    try:
        import importlib
        mod = importlib.import_module(root)
    except Exception:
        return result
    conv = getattr(mod, "from_dlpack", None)
    return conv(result) if conv is not None else result


def _as_tensor(a, dtype, name):
    torch = _torch()
    if not isinstance(a, torch.Tensor):
        a = torch.from_dlpack(a) if hasattr(a, "__dlpack__") else torch.as_tensor(a, device="cuda")
    if not a.is_cuda:
        raise ValueError("%s must be a CUDA array" % name)
    if a.dtype != dtype:
        raise ValueError("%s must have dtype %s (got %s)" % (name, dtype, a.dtype))
    if a.dim() != 1:
        raise ValueError("%s must be one-dimensional" % name)
    return a.contiguous()


def _enter(ctx, ref):
    """Bind the context to the caller's current stream so that work queued by the
    caller before the call is ordered before ours."""
    torch = _torch()
    stream = torch.cuda.current_stream(ref.device).cuda_stream
    # handle 0 is the legacy default stream; the C ABI wants its explicit name (0x1)
    _lib.load().sporder_context_set_stream(ctx.handle, C.c_void_p(stream if stream else 1))


def _sizes(ptr, ind):
    if ptr.numel() < 2:
        raise ValueError("ptr must have length n+1 (at least 2)")
    n, nnz = ptr.numel() - 1, ind.numel()
    if n > 2**31 - 1 or nnz > 2**31 - 1:
        raise ValueError("matrix too large for int32 indexing")
    return n, nnz


def _timing_dict(t):
    return {"wall_ms": t.wall_ms, "csr2csc_ms": t.csr2csc_ms, "similarity_ms": t.similarity_ms,
            "chunk_greedy_ms": t.chunk_greedy_ms}


def _stats_dict(s):
    return {f: getattr(s, f) for f, _ in s._fields_}


def chunk_similarity_greedy(ptr, ind, *, is_symmetric=False, k=0, oversampling=0.0, chunk_size=0,
                            with_timing=False, with_stats=False, ctx=None):
    """One-shot per-chunk similarity + greedy seriation
    (sporder/python/sporder/__init__.py:380-424).

    Returns ``new_order`` (int32 CUDA tensor, new2old); a ``timing`` dict (wall_ms,
    csr2csc_ms, similarity_ms, chunk_greedy_ms) and/or a ``stats`` dict (k_used, m_used,
    avg_degree, avg_edge_weight, zero_degree_rows, chunk_size_used, chain_restarts,
    avg_followed_weight) are appended when requested."""
    torch = _torch()
    src = ptr
    ptr = _as_tensor(ptr, torch.int32, "ptr")
    ind = _as_tensor(ind, torch.int32, "ind")
    n, nnz = _sizes(ptr, ind)
    ctx = _ctx(ctx, ptr)
    lib = _lib.load()
    with torch.cuda.device(ptr.device):
        _enter(ctx, ptr)
        order = torch.empty(n, dtype=torch.int32, device=ptr.device)
        timing, stats = _lib.CsgTiming(), _lib.CsgStats()
        lib.sporder_chunk_similarity_greedy(
            ctx.handle, n, nnz, ptr.data_ptr(), ind.data_ptr(), bool(is_symmetric), int(k),
            float(oversampling), int(chunk_size), order.data_ptr(),
            C.byref(timing) if with_timing else None, C.byref(stats) if with_stats else None)
    msg = _lib.last_error()
    if msg:
        raise ValueError(msg) if "expect" in msg or "must be" in msg else RuntimeError(msg)
    result = (_like(order, src),)
    if with_timing:
        result += (_timing_dict(timing),)
    if with_stats:
        result += (_stats_dict(stats),)
    return result if len(result) > 1 else result[0]


def csg_table(ptr, ind, *, is_symmetric=False, k=0, oversampling=0.0, chunk_size=0,
              with_order=True, ctx=None):
    """csg that also returns the top-k candidate table: ``(order, table)`` with
    ``table`` an ``(n, k_used)`` int64 tensor of packed entries (high word = fp32 bits
    of the weight, low word = index + 1, 0 = empty).  No reference counterpart: the
    reference never exposes this table."""
    torch = _torch()
    src = ptr
    ptr = _as_tensor(ptr, torch.int32, "ptr")
    ind = _as_tensor(ind, torch.int32, "ind")
    n, nnz = _sizes(ptr, ind)
    ctx = _ctx(ctx, ptr)
    lib = _lib.load()
    kk = int(k) if k > 0 else min(256, max(16, nnz // n))
    with torch.cuda.device(ptr.device):
        _enter(ctx, ptr)
        order = torch.empty(n, dtype=torch.int32, device=ptr.device) if with_order else None
        table = torch.empty((n, kk), dtype=torch.int64, device=ptr.device)
        k_used = lib.sporder_csg_with_table(
            ctx.handle, n, nnz, ptr.data_ptr(), ind.data_ptr(), bool(is_symmetric), int(k),
            float(oversampling), int(chunk_size), order.data_ptr() if with_order else None,
            table.data_ptr(), table.numel(), None, None)
    msg = _lib.last_error()
    if msg:
        raise ValueError(msg) if "expect" in msg or "must be" in msg else RuntimeError(msg)
    assert k_used == kk
    return _like(order, src), _like(table, src)


def chunk_similarity_greedy_host(ptr, ind, *, is_symmetric=False, k=0, oversampling=0.0,
                                 chunk_size=0, out=None, ctx=None):
    """csg on HOST int32 tensors (pinned for full copy speed): copies the pattern to
    the device, reorders, copies the permutation back into ``out`` (a host int32
    tensor, allocated pinned when None).  No reference counterpart."""
    torch = _torch()
    if ptr.is_cuda or ind.is_cuda or ptr.dtype != torch.int32 or ind.dtype != torch.int32:
        raise ValueError("ptr and ind must be int32 host tensors")
    n, nnz = _sizes(ptr, ind)
    ctx = _ctx(ctx, ptr)
    if out is None:
        out = torch.empty(n, dtype=torch.int32).pin_memory()
    lib = _lib.load()
    lib.sporder_context_set_stream(ctx.handle, None)
    rc = lib.sporder_chunk_similarity_greedy_host(
        ctx.handle, n, nnz, ptr.data_ptr(), ind.data_ptr(), bool(is_symmetric), int(k),
        float(oversampling), int(chunk_size), out.data_ptr(), None, None)
    if rc != 0:
        _lib.check()
    return out


def chunk_greedy(ptr, ind, *, is_symmetric=False, k=0, oversampling=0.0, chunk_size=0,
                 with_timing=False, with_stats=False, ctx=None):
    """Chunked greedy seriation on the GLOBAL top-k graph (the reference's ``cg``;
    sporder/include/sporder.h:169-182): ``new_order`` [, timing dict] [, stats dict with
    the csg fields plus ``cut_weight_fraction``]."""
    torch = _torch()
    src = ptr
    ptr = _as_tensor(ptr, torch.int32, "ptr")
    ind = _as_tensor(ind, torch.int32, "ind")
    n, nnz = _sizes(ptr, ind)
    ctx = _ctx(ctx, ptr)
    lib = _lib.load()
    with torch.cuda.device(ptr.device):
        _enter(ctx, ptr)
        order = torch.empty(n, dtype=torch.int32, device=ptr.device)
        timing, stats = _lib.CsgTiming(), _lib.CgStats()
        lib.sporder_chunk_greedy(
            ctx.handle, n, nnz, ptr.data_ptr(), ind.data_ptr(), bool(is_symmetric), int(k),
            float(oversampling), int(chunk_size), order.data_ptr(),
            C.byref(timing) if with_timing else None, C.byref(stats) if with_stats else None)
    msg = _lib.last_error()
    if msg:
        raise ValueError(msg) if "expect" in msg or "must be" in msg else RuntimeError(msg)
    result = (_like(order, src),)
    if with_timing:
        result += (_timing_dict(timing),)
    if with_stats:
        result += ({f: getattr(stats, f) for f, _ in _lib.CgStats._fields_},)
    return result if len(result) > 1 else result[0]


def similarity_graph(ptr, ind, *, is_symmetric=False, k=0, oversampling=0.0, with_timing=False,
                     with_stats=False, ctx=None):
    """Weighted top-k Dice-similarity graph (sporder/python/sporder/__init__.py:200-259):
    ``(indices, weights)``, two ``(n, k_used)`` CUDA tensors (int32 / float32), entries by
    descending weight per row, unused entries index -1 and weight 0; a ``timing`` dict
    (wall_ms, csr2csc_ms, similarity_ms, unpack_ms) and/or a ``stats`` dict (k_used, m_used,
    avg_degree, avg_edge_weight, zero_degree_rows) are appended when requested."""
    torch = _torch()
    src = ptr
    ptr = _as_tensor(ptr, torch.int32, "ptr")
    ind = _as_tensor(ind, torch.int32, "ind")
    n, nnz = _sizes(ptr, ind)
    kk = int(k) if k > 0 else min(32, max(16, 2 * (nnz // max(n, 1))))  # sporder.cpp:75-77
    ctx = _ctx(ctx, ptr)
    lib = _lib.load()
    with torch.cuda.device(ptr.device):
        _enter(ctx, ptr)
        idx = torch.empty((n, kk), dtype=torch.int32, device=ptr.device)
        wgt = torch.empty((n, kk), dtype=torch.float32, device=ptr.device)
        timing, stats = _lib.SimTiming(), _lib.SimStats()
        rc = lib.sporder_similarity_graph(
            ctx.handle, n, nnz, ptr.data_ptr(), ind.data_ptr(), bool(is_symmetric), kk,
            float(oversampling), idx.data_ptr(), wgt.data_ptr(),
            C.byref(timing) if with_timing else None, C.byref(stats) if with_stats else None)
    if rc < 0:
        msg = _lib.last_error() or "sporder_similarity_graph failed"
        raise ValueError(msg) if "expect" in msg or "must be" in msg else RuntimeError(msg)
    result = (_like(idx, src), _like(wgt, src))
    if with_timing:
        result += (dict(wall_ms=timing.wall_ms, csr2csc_ms=timing.csr2csc_ms,
                        similarity_ms=timing.similarity_ms, unpack_ms=timing.unpack_ms),)
    if with_stats:
        result += (dict(k_used=stats.k_used, m_used=stats.m_used, avg_degree=stats.avg_degree,
                        avg_edge_weight=stats.avg_edge_weight,
                        zero_degree_rows=stats.zero_degree_rows),)
    return result


def count_pillars(ptr, ind, height, *, ctx=None):
    """Distinct (row // height, column) pairs of a CSR pattern: the reference's reordering
    quality metric, fewer is better (sporder/python/sporder/__init__.py:152-172)."""
    torch = _torch()
    src = ptr
    ptr = _as_tensor(ptr, torch.int32, "ptr")
    ind = _as_tensor(ind, torch.int32, "ind")
    n, nnz = _sizes(ptr, ind)
    if int(height) < 1:
        raise ValueError("height must be >= 1")
    ctx = _ctx(ctx, ptr)
    lib = _lib.load()
    out = C.c_int32(0)
    with torch.cuda.device(ptr.device):
        _enter(ctx, ptr)
        lib.sporder_count_pillars(ctx.handle, n, nnz, ptr.data_ptr(), ind.data_ptr(), int(height),
                                  C.byref(out))
    _lib.check()
    return int(out.value)


def reorder(ptr, ind, new_order, *, val=None, symmetric=False, ctx=None):
    """Apply a row (or symmetric row+column) permutation to a CSR pattern
    (sporder/python/sporder/__init__.py:113-149).  Returns ``(ptr_new, ind_new)`` or
    ``(ptr_new, ind_new, val_new)``; column indices are sorted inside each row."""
    torch = _torch()
    src = ptr
    ptr = _as_tensor(ptr, torch.int32, "ptr")
    ind = _as_tensor(ind, torch.int32, "ind")
    new_order = _as_tensor(new_order, torch.int32, "new_order")
    n, nnz = _sizes(ptr, ind)
    if new_order.numel() != n:
        raise ValueError("new_order must have length n")
    if val is not None:
        val = _as_tensor(val, torch.float32, "val")
        if val.device != ptr.device:
            raise ValueError("val must live on the same device as ptr")
        if val.numel() != nnz:
            raise ValueError("val must have length nnz")
    ctx = _ctx(ctx, ptr)
    lib = _lib.load()
    with torch.cuda.device(ptr.device):
        _enter(ctx, ptr)
        ptr_new = torch.empty(n + 1, dtype=torch.int32, device=ptr.device)
        ind_new = torch.empty(max(nnz, 1), dtype=torch.int32, device=ptr.device)[:nnz]
        val_new = None
        if val is not None:
            val_new = torch.empty(max(nnz, 1), dtype=torch.float32, device=ptr.device)[:nnz]
        lib.sporder_reorder(ctx.handle, n, nnz, ptr.data_ptr(), ind.data_ptr(),
                            val.data_ptr() if val is not None else None, new_order.data_ptr(),
                            1 if symmetric else 0, ptr_new.data_ptr(), ind_new.data_ptr(),
                            val_new.data_ptr() if val is not None else None)
    _lib.check()
    out = (ptr_new, ind_new) if val is None else (ptr_new, ind_new, val_new)
    return tuple(_like(a, src) for a in out)


def spmm(ptr, ind, val, B, *, out=None, sync=True, ctx=None, n_cols=None):
    """fp32 CSR SpMM ``C = A @ B`` with ``B`` a row-major ``(n, w)`` float32 CUDA
    tensor.  The reference has no first-party SpMM (it times third-party kernels,
    bench/spmm/spmm_bench/base.py:48-59); this is the kernel the reordered matrix is
    fed to.  ``sync=False`` skips the final stream synchronisation.  ``n_cols`` names the
    column count of a row block cut out of a wider matrix (the row-partitioned multi-GPU
    product): ``B`` then has ``n_cols`` rows and ``C`` as many rows as the block."""
    torch = _torch()
    src = ptr
    ptr = _as_tensor(ptr, torch.int32, "ptr")
    ind = _as_tensor(ind, torch.int32, "ind")
    val = _as_tensor(val, torch.float32, "val")
    n, nnz = _sizes(ptr, ind)
    if not isinstance(B, torch.Tensor):
        B = torch.from_dlpack(B)
    rows_b = n if n_cols is None else int(n_cols)
    if B.dim() != 2 or B.shape[0] != rows_b or B.dtype != torch.float32 or not B.is_cuda:
        raise ValueError("B must be a float32 CUDA tensor of shape (%d, w)" % rows_b)
    B = B.contiguous()
    w = B.shape[1]
    ctx = _ctx(ctx, ptr)
    lib = _lib.load()
    with torch.cuda.device(ptr.device):
        _enter(ctx, ptr)
        if out is None:
            out = torch.empty((n, w), dtype=torch.float32, device=ptr.device)
        fn = lib.sporder_spmm if sync else lib.sporder_spmm_async
        rc = fn(ctx.handle, n, nnz, w, ptr.data_ptr(), ind.data_ptr(), val.data_ptr(),
                B.data_ptr(), out.data_ptr())
    if rc != 0:
        _lib.check()
    return _like(out, src)


def kernel_launches():
    """Kernels launched by the library in this process so far."""
    return int(_lib.load().sporder_kernel_launches())
