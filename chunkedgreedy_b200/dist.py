"""Row sharding of the csg path over the GPUs of one node.

Every chunk of ``chunk_size`` consecutive rows is an independent problem for the
sketch, the top-k and the greedy stage (sporder/src/common/chunk_similarity_top_k.cu:46-50,71;
sporder/src/csg/chunk_similarity_greedy.cu:18-24), and the in-chunk part of every column
list can be derived from the chunk's own rows.  A shard made of whole chunks therefore needs
no data from other shards: each rank reorders its row block with the single-GPU kernels
(``sporder_csg_shard``) and the only exchange is an all-gather of the permutation shards
(4 bytes per row).  The SpMM that follows the reorder shards by rows as well: every rank
multiplies a contiguous, nonzero-balanced row range of the matrix with the whole dense
operand (replicated) and owns that row range of the result; the result is all-gathered only
when the next operation needs it whole (a GCN layer feeding the next propagation).  The
reference has no multi-GPU mode; this module is new surface.

Host logic here is backend-neutral (it runs under ``gloo`` on CPU in the tests with a
stand-in for the per-shard compute); the product path calls the CUDA library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

__all__ = ["shard_bounds", "extract_shard", "gather_shards", "csg_shard",
           "chunk_similarity_greedy_sharded", "resolve_k", "spmm_row_bounds", "spmm_shard",
           "spmm_sharded"]


def resolve_k(n, nnz, k=0):
    """k of the whole matrix (sporder/src/sporder.cpp:147-149); shards must all use it."""
    return int(k) if k > 0 else min(256, max(16, nnz // n))


def shard_bounds(ptr, chunk_size, world_size):
    """Chunk-aligned row ranges ``[(r0, r1), ...]``, one per rank, balanced by nonzeros.

    ``ptr`` is the full row-pointer array (numpy or torch, host).  Ranks may get an empty
    range when there are fewer chunks than ranks."""
    ptr = np.asarray(ptr)
    n = ptr.size - 1
    chunk_size = int(chunk_size) if chunk_size > 0 else 1024
    num_chunks = (n + chunk_size - 1) // chunk_size
    edges = np.minimum(np.arange(num_chunks + 1, dtype=np.int64) * chunk_size, n)
    cum = ptr[edges].astype(np.int64)  # nonzeros before each chunk boundary
    total = int(cum[-1])
    cuts = [0]
    for r in range(1, world_size):
        target = total * r / world_size
        c = int(np.searchsorted(cum, target, side="left"))
        # nearest boundary, never moving backwards
        if c > 0 and abs(cum[c - 1] - target) <= abs(cum[min(c, num_chunks)] - target):
            c -= 1
        cuts.append(min(max(c, cuts[-1]), num_chunks))
    cuts.append(num_chunks)
    return [(int(edges[cuts[i]]), int(edges[cuts[i + 1]])) for i in range(world_size)]


def extract_shard(ptr, ind, r0, r1):
    """Rows ``[r0, r1)`` as a CSR block with the row pointers rebased to 0 (numpy views /
    small copies; the column ids stay those of the full matrix)."""
    ptr = np.asarray(ptr)
    b, e = int(ptr[r0]), int(ptr[r1])
    return (ptr[r0:r1 + 1] - ptr[r0]).astype(np.int32), np.asarray(ind)[b:e]


def gather_shards(local, bounds, group=None):
    """All-gather per-rank 1-D tensors of unequal length into one tensor ordered by rank.

    Shards are padded to the longest one (one collective, no size exchange: every rank
    knows ``bounds``)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = [r1 - r0 for r0, r1 in bounds]
    longest = max(max(sizes), 1)
    buf = torch.zeros(longest, dtype=local.dtype, device=local.device)
    buf[: local.numel()] = local
    out = torch.empty(world * longest, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, buf, group=group)
    if all(s == longest for s in sizes):
        return out
    return torch.cat([out[i * longest: i * longest + sizes[i]] for i in range(world)])


def csg_shard(ptr_local, ind_local, n_cols, row_base, *, k, oversampling=0.0, chunk_size=0,
              with_table=False, with_timing=False, with_stats=False, ctx=None):
    """Reorder one row shard on the current CUDA device (``sporder_csg_shard``).

    ``ptr_local`` / ``ind_local``: int32 CUDA tensors of the block (pointers rebased to 0).
    Returns the block's slice of the global permutation [, its table rows] [, timing]
    [, statistics of the block]."""
    import torch
    from . import _ctx, _enter, _lib, _stats_dict, _timing_dict
    n_rows, nnz = ptr_local.numel() - 1, ind_local.numel()
    if k <= 0:
        raise ValueError("csg_shard needs the matrix-wide k (see resolve_k)")
    ctx = _ctx(ctx, ptr_local)
    lib = _lib.load()
    order = torch.empty(max(n_rows, 0), dtype=torch.int32, device=ptr_local.device)
    table = torch.empty((n_rows, k), dtype=torch.int64, device=ptr_local.device) if with_table else None
    timing, stats = _lib.CsgTiming(), _lib.CsgStats()
    if n_rows > 0:
        with torch.cuda.device(ptr_local.device):
            _enter(ctx, ptr_local)
            rc = lib.sporder_csg_shard(
                ctx.handle, n_rows, int(n_cols), int(row_base), nnz, ptr_local.data_ptr(),
                ind_local.data_ptr(), int(k), float(oversampling), int(chunk_size),
                order.data_ptr(), table.data_ptr() if with_table else None,
                table.numel() if with_table else 0, C.byref(timing) if with_timing else None,
                C.byref(stats) if with_stats else None)
        if rc < 0:
            _lib.check()
    out = (order,)
    if with_table:
        out += (table,)
    if with_timing:
        out += (_timing_dict(timing),)
    if with_stats:
        out += (_stats_dict(stats),)
    return out if len(out) > 1 else out[0]


def chunk_similarity_greedy_sharded(ptr, ind, *, k=0, oversampling=0.0, chunk_size=0, group=None,
                                    compute=None, device=None):
    """csg over all ranks of ``group``: every rank passes the SAME full host CSR
    (numpy int32), takes its chunk-aligned block, reorders it and receives the whole
    permutation.  ``compute(ptr_local, ind_local, n_cols, row_base, k, oversampling,
    chunk_size) -> 1-D tensor`` replaces the CUDA call (used by the CPU tests)."""
    import torch
    import torch.distributed as dist
    ptr = np.asarray(ptr)
    n, nnz = ptr.size - 1, int(np.asarray(ind).size)
    chunk = int(chunk_size) if chunk_size > 0 else 1024
    kk = resolve_k(n, nnz, k)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    bounds = shard_bounds(ptr, chunk, world)
    r0, r1 = bounds[rank]
    pl, il = extract_shard(ptr, ind, r0, r1)
    if compute is None:
        device = device or torch.device("cuda", torch.cuda.current_device())
        dp = torch.from_numpy(np.ascontiguousarray(pl)).to(device)
        di = torch.from_numpy(np.ascontiguousarray(il)).to(device)
        local = csg_shard(dp, di, n, r0, k=kk, oversampling=oversampling, chunk_size=chunk)
    else:
        local = compute(pl, il, n, r0, kk, oversampling, chunk)
    return gather_shards(local, bounds, group)


SPMM_ROW_COST = 4  # what a row costs the SpMM kernel beside its nonzeros, in nonzeros


def spmm_row_bounds(ptr, world_size):
    """Contiguous row ranges ``[(r0, r1), ...]`` for the row-partitioned SpMM, one per rank,
    balanced by the kernel's own cost measure, nonzeros plus ``SPMM_ROW_COST`` per row (no
    chunk alignment: SpMM rows are independent; balancing nonzeros alone gives the rank with
    the hub rows too little and the rank with the many short rows too much to do).  ``ptr``
    may be a numpy array or a (host or device) torch tensor."""
    if hasattr(ptr, "detach"):
        ptr = ptr.detach().cpu().numpy()
    ptr = np.asarray(ptr)
    n = ptr.size - 1
    cost = ptr.astype(np.int64) + SPMM_ROW_COST * np.arange(n + 1, dtype=np.int64)
    total = int(cost[-1])
    cuts = [0]
    for r in range(1, world_size):
        c = int(np.searchsorted(cost, total * r / world_size, side="left"))
        cuts.append(min(max(c, cuts[-1]), n))
    cuts.append(n)
    return [(cuts[i], cuts[i + 1]) for i in range(world_size)]


def spmm_shard(ptr, ind, val, r0, r1):
    """Rows ``[r0, r1)`` of a CSR matrix held in torch tensors as a CSR block: rebased row
    pointers (a small new tensor) and views of the index and value arrays."""
    b, e = int(ptr[r0]), int(ptr[r1])
    return (ptr[r0:r1 + 1] - ptr[r0]).contiguous(), ind[b:e], val[b:e]


def spmm_sharded(ptr, ind, val, B, *, bounds=None, gather=False, group=None, compute=None,
                 out=None, ctx=None, sync=True):
    """Row-partitioned ``C = A @ B`` over the ranks of ``group``: every rank holds the matrix
    (``ptr``, ``ind``, ``val``: torch tensors, the SAME on every rank) and the whole dense
    operand ``B``; it multiplies its own nonzero-balanced row range and returns that block of
    ``C`` (shape ``(r1 - r0, w)``), or the whole ``C`` after one all-gather when
    ``gather=True``.  No kernel ever reads another GPU's memory.

    ``compute(ptr_local, ind_local, val_local, B) -> (rows, w) tensor`` replaces the CUDA
    kernel (used by the CPU tests)."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if bounds is None:
        bounds = spmm_row_bounds(ptr, world)
    r0, r1 = bounds[rank]
    w = B.shape[1]
    if r1 > r0:
        pl, il, vl = spmm_shard(ptr, ind, val, r0, r1)
        if compute is None:
            from . import spmm
            local = spmm(pl, il, vl, B, n_cols=B.shape[0], out=out, ctx=ctx, sync=sync)
        else:
            local = compute(pl, il, vl, B)
    else:
        local = torch.empty((0, w), dtype=B.dtype, device=B.device)
    if not gather:
        return local
    flat = gather_shards(local.reshape(-1), [(a * w, b * w) for a, b in bounds], group)
    return flat.reshape(-1, w)
