"""Method module for the reference's reorder harness, with torch in place of CuPy.

Shaped like bench/reorder/reorder_bench/methods/sporder_csg.py:25-70: ``reorder(csr, params)``
takes a scipy CSR matrix and the method's parameters (``k``, ``oversampling``,
``chunk_size``, optional ``auto_detect_symmetric``) and returns the row permutation with
the harness's timings -- preparation (sort indices, symmetry check, upload:
reorder_bench/loader.py:63-93), the library's own ``wall_ms`` of the second call after an
untimed warm-up call and an L2 flush (reorder_bench/timing.py:29-41), and its stage
breakdown.  When the harness package is importable the result is its ``ReorderResult``;
otherwise a dataclass with the same fields, so the module can be used and tested alone.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any

import numpy as np

__all__ = ["reorder", "ReorderResult", "prep_gpu", "flush_l2", "B200SpMM", "amortization_runs",
           "format_amortization"]


try:  # the harness's own result type, when this runs inside the harness
    from reorder_bench.types import ReorderResult  # type: ignore
except Exception:  # pragma: no cover - the harness is not part of this repository
    @dataclass
    class ReorderResult:  # fields of reorder_bench/types.py:10-17
        row_perm: np.ndarray
        reorder_time_ms: float
        prep_time_ms: float = 0.0
        perm_trans_ms: float = 0.0
        timing_breakdown: dict = field(default_factory=dict)
        effective_params: dict = field(default_factory=dict)
        env_extra: dict = field(default_factory=dict)


def prep_gpu(csr, detect_symmetric=True, device=None):
    """Sorted int32 ptr/ind on the GPU, the symmetry flag and the time it took
    (reorder_bench/loader.py:63-93)."""
    import torch
    int32_max = np.iinfo(np.int32).max
    nrows, nnz = int(csr.shape[0]), int(csr.nnz)
    if nrows > int32_max or nnz > int32_max:
        raise ValueError("matrix does not fit 32-bit indices: %d rows, %d nonzeros" % (nrows, nnz))
    device = device or torch.device("cuda", torch.cuda.current_device())
    t0 = time.perf_counter()
    out = csr.copy()
    out.sort_indices()
    is_symmetric = bool((out != out.T).nnz == 0) if detect_symmetric else False
    ptr = torch.from_numpy(np.ascontiguousarray(out.indptr, dtype=np.int32)).to(device)
    ind = torch.from_numpy(np.ascontiguousarray(out.indices, dtype=np.int32)).to(device)
    torch.cuda.synchronize(device)
    return ptr, ind, is_symmetric, (time.perf_counter() - t0) * 1e3


def flush_l2(device=None):
    """Writes a buffer twice the size of L2 (reorder_bench/timing.py:29-41)."""
    import torch
    device = device or torch.device("cuda", torch.cuda.current_device())
    l2 = torch.cuda.get_device_properties(device).L2_cache_size or 6 * 1024 * 1024
    buf = torch.empty(int(l2) * 2, dtype=torch.uint8, device=device)
    buf.zero_()
    torch.cuda.synchronize(device)


def reorder(csr, params: dict[str, Any]) -> ReorderResult:
    import chunkedgreedy_b200 as lib
    want_symmetry_check = bool(params.get("auto_detect_symmetric", True))
    d_ptr, d_ind, symmetric, upload_ms = prep_gpu(csr, detect_symmetric=want_symmetry_check)
    options = dict(is_symmetric=symmetric, k=int(params.get("k", 0)),
                   oversampling=float(params.get("oversampling", 0.0)),
                   chunk_size=int(params.get("chunk_size", 0)))
    # the harness's protocol: one untimed call, a flushed L2, then the library's own wall time
    lib.chunk_similarity_greedy(d_ptr, d_ind, **options)
    flush_l2(d_ptr.device)
    new2old, t = lib.chunk_similarity_greedy(d_ptr, d_ind, with_timing=True, **options)
    t0 = time.perf_counter()
    perm = new2old.cpu().numpy().astype(np.int64)
    if perm.shape[0] != csr.shape[0]:
        raise ValueError("perm length %d != nrows %d" % (perm.shape[0], csr.shape[0]))
    to_host_ms = (time.perf_counter() - t0) * 1e3
    stages = {name: float(t.get(name, 0.0)) for name in ("csr2csc_ms", "similarity_ms", "chunk_greedy_ms")}
    return ReorderResult(row_perm=perm, reorder_time_ms=float(t["wall_ms"]), prep_time_ms=upload_ms,
                         perm_trans_ms=to_host_ms, timing_breakdown=stages,
                         effective_params={"is_symmetric": symmetric})


def amortization_runs(reorder_time_ms, spmm_original_ms, spmm_reordered_ms):
    """SpMM launches after which a reorder has paid for itself: reorder time over the time
    one launch saves; infinite when the reordered matrix is not faster
    (bench/spmm/scripts/compute_amortization.py:63-66)."""
    saved = float(spmm_original_ms) - float(spmm_reordered_ms)
    if saved <= 0:
        return float("inf")
    return float(reorder_time_ms) / saved


def format_amortization(value):
    """The harness's text form (compute_amortization.py:48-51): "inf" or ten significant digits."""
    return "inf" if value == float("inf") else "%.10g" % value


try:  # the harness's base class, when this runs inside the harness
    from spmm_bench.base import SpMMMethod as _SpMMBase  # type: ignore
except Exception:  # pragma: no cover - the harness is not part of this repository
    _SpMMBase = object


class B200SpMM(_SpMMBase):
    """This library's fp32 CSR SpMM as a method of the reference's SpMM harness
    (bench/spmm/spmm_bench/base.py:8-65): ``build`` / ``prepare`` / ``run``, where ``run``
    makes exactly one timed launch and returns ``(C, kernel_ms)`` measured with CUDA events
    around the kernel only; warm-up and averaging are the caller's."""

    @property
    def name(self) -> str:
        return "sporder-b200-spmm"

    @property
    def uses_feature_dim(self) -> bool:
        return True

    @property
    def uses_cuda(self) -> bool:
        return True

    @property
    def tc_h(self) -> int:  # no tensor-core tiles: plain fp32 rows
        return 1

    @property
    def tc_w(self) -> int:
        return 1

    def build(self) -> None:
        from . import _lib
        try:
            _lib.load()
        except Exception as exc:
            raise RuntimeError("sporder_b200 library not built: %s" % exc) from exc

    def prepare(self, A_csr):
        """scipy CSR -> (ptr, ind, val) int32/int32/float32 CUDA tensors (untimed)."""
        import torch
        out = A_csr.copy()
        out.sort_indices()
        dev = torch.device("cuda", torch.cuda.current_device())
        ptr = torch.from_numpy(np.ascontiguousarray(out.indptr, dtype=np.int32)).to(dev)
        ind = torch.from_numpy(np.ascontiguousarray(out.indices, dtype=np.int32)).to(dev)
        val = torch.from_numpy(np.ascontiguousarray(out.data, dtype=np.float32)).to(dev)
        return ptr, ind, val

    def run(self, prepared_A, B):
        import torch
        import chunkedgreedy_b200 as sporder
        ptr, ind, val = prepared_A
        B = B.contiguous().to(torch.float32)
        C = torch.empty((ptr.numel() - 1, B.shape[1]), dtype=torch.float32, device=B.device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        sporder.spmm(ptr, ind, val, B, out=C, sync=False)
        e1.record()
        torch.cuda.synchronize(B.device)
        return C, float(e0.elapsed_time(e1))
