"""Row sharding on CPU: bounds, block extraction and the gloo all-gather, with the
oracle standing in for the per-shard CUDA call (world_size 2 and 3)."""
import os
import socket

import numpy as np
import pytest

import cases
import oracle
from chunkedgreedy_b200 import dist as csgdist

torch = pytest.importorskip("torch")


def test_shard_bounds_are_chunk_aligned_and_cover():
    ptr, ind, val, sym, params = cases.build("rmat12")
    n = ptr.size - 1
    for world in (1, 2, 3, 4, 8, 16):
        b = csgdist.shard_bounds(ptr, 1024, world)
        assert len(b) == world and b[0][0] == 0 and b[-1][1] == n
        for (a0, a1), (b0, b1) in zip(b, b[1:]):
            assert a1 == b0
        for r0, r1 in b:
            assert r0 % 1024 == 0 and (r1 % 1024 == 0 or r1 == n) and r0 <= r1


def test_shard_bounds_balance_nonzeros():
    ptr, ind, val, sym, params = cases.build("zipf65k")
    b = csgdist.shard_bounds(ptr, 1024, 4)
    nnz = [int(ptr[r1] - ptr[r0]) for r0, r1 in b]
    assert max(nnz) <= 1.3 * (sum(nnz) / 4)


def test_shards_reproduce_the_full_problem_serially():
    # every shard alone gives its slice of the full answer (orders and tables)
    ptr, ind, val, sym, params = cases.build("rmat12")
    n = ptr.size - 1
    k = csgdist.resolve_k(n, ind.size)
    full_order, full_table = oracle.csg(ptr, ind, False, with_table=True)
    for r0, r1 in csgdist.shard_bounds(ptr, 1024, 3):
        if r1 == r0:
            continue
        pl, il = csgdist.extract_shard(ptr, ind, r0, r1)
        o, t = oracle.csg(pl, il, False, k=k, with_table=True, ncols=n)
        assert np.array_equal(o + r0, full_order[r0:r1])
        idx, w = oracle.decode_table(t)
        fidx, fw = oracle.decode_table(full_table[r0:r1])
        assert np.array_equal(np.where(idx >= 0, idx + r0, -1), fidx) and np.array_equal(w, fw)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, name, result_path):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ptr, ind, val, sym, params = cases.build(name)

    def compute(pl, il, n_cols, row_base, k, ovs, chunk):
        if pl.size <= 1:
            return torch.empty(0, dtype=torch.int32)
        o = oracle.csg(pl, il, False, k=k, oversampling=ovs, chunk_size=chunk, ncols=n_cols)
        return torch.from_numpy(o + np.int32(row_base))

    order = csgdist.chunk_similarity_greedy_sharded(ptr, ind, compute=compute, **params)
    if rank == 0:
        np.save(result_path, order.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,name", [(2, "rmat12"), (3, "hub_c700"), (2, "tiny1")])
def test_gloo_sharded_csg_equals_single_process(world, name, tmp_path):
    import torch.multiprocessing as mp
    ptr, ind, val, sym, params = cases.build(name)
    path = str(tmp_path / "order.npy")
    mp.spawn(_worker, args=(world, _free_port(), name, path), nprocs=world, join=True)
    got = np.load(path)
    assert np.array_equal(got, oracle.csg(ptr, ind, False, **params))


def test_spmm_row_bounds_cover_and_balance():
    ptr, ind, val, sym, params = cases.build("zipf65k")
    n = ptr.size - 1
    for world in (1, 2, 3, 8):
        b = csgdist.spmm_row_bounds(ptr, world)
        assert len(b) == world and b[0][0] == 0 and b[-1][1] == n
        assert all(a1 == b0 for (_, a1), (b0, _) in zip(b, b[1:]))
        cost = [int(ptr[r1] - ptr[r0]) + csgdist.SPMM_ROW_COST * (r1 - r0) for r0, r1 in b]
        assert max(cost) <= 1.2 * (sum(cost) / world) + 4096 + csgdist.SPMM_ROW_COST
    # more ranks than rows: the extra ranks get empty ranges
    b = csgdist.spmm_row_bounds(np.array([0, 2, 3], dtype=np.int32), 5)
    assert b[0][0] == 0 and b[-1][1] == 2 and sum(r1 - r0 for r0, r1 in b) == 2


def _spmm_worker(rank, world, port, name, w, result_path):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ptr, ind, val, sym, params = cases.build(name)
    n = ptr.size - 1
    B = np.random.default_rng(5).standard_normal((n, w)).astype(np.float32)

    def compute(pl, il, vl, Bt):  # the CPU restatement in place of the CUDA kernel
        return torch.from_numpy(oracle.spmm_f32(pl.numpy(), il.numpy(), vl.numpy(), Bt.numpy()))

    tp, ti, tv = torch.from_numpy(ptr), torch.from_numpy(ind), torch.from_numpy(val)
    local = csgdist.spmm_sharded(tp, ti, tv, torch.from_numpy(B), compute=compute)
    r0, r1 = csgdist.spmm_row_bounds(ptr, world)[rank]
    assert tuple(local.shape) == (r1 - r0, w)
    whole = csgdist.spmm_sharded(tp, ti, tv, torch.from_numpy(B), compute=compute, gather=True)
    if rank == 0:
        np.save(result_path, whole.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,name,w", [(2, "rmat12", 8), (3, "ragged", 5), (2, "tiny1", 3)])
def test_gloo_row_partitioned_spmm_equals_single_process(world, name, w, tmp_path):
    import torch.multiprocessing as mp
    ptr, ind, val, sym, params = cases.build(name)
    n = ptr.size - 1
    path = str(tmp_path / "c.npy")
    mp.spawn(_spmm_worker, args=(world, _free_port(), name, w, path), nprocs=world, join=True)
    B = np.random.default_rng(5).standard_normal((n, w)).astype(np.float32)
    got = np.load(path)
    assert got.shape == (n, w)
    assert np.array_equal(got, oracle.spmm_f32(ptr, ind, val, B))  # same kernel, same order of adds
    c64, cabs = oracle.spmm_f64(ptr, ind, val, B)
    assert np.all(np.abs(got - c64) <= 1e-5 * cabs + 1e-30)
