"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle, the
committed reference outputs and (when its build travelled with the repository) the
reference's own CUDA library.  Bit-exact for tables, permutations and reordered
matrices; SpMM within 1e-5 of the fp64 product, scaled by sum_j |a_ij * b_jl|."""
import hashlib
import os

import numpy as np
import pytest

import cases
import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _sp():
    import chunkedgreedy_b200 as sp
    return sp


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8)


@pytest.mark.parametrize("name", list(cases.CASES))
def test_csg_matches_reference_outputs_and_oracle(name, golden):
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    order, table = sp.csg_table(_dev(ptr), _dev(ind), is_symmetric=sym, **params)
    order, table = order.cpu().numpy(), table.cpu().numpy().view(np.uint64)
    o_or, t_or = oracle.csg(ptr, ind, sym, with_table=True, **params)
    assert np.array_equal(table, t_or)
    assert np.array_equal(order, o_or)
    assert np.array_equal(order, golden[name + "/order"])
    assert np.array_equal(_sha(table), golden[name + "/table_sha256"])
    plain = sp.chunk_similarity_greedy(_dev(ptr), _dev(ind), is_symmetric=sym, **params)
    assert np.array_equal(plain.cpu().numpy(), o_or)


@pytest.mark.parametrize("name", list(cases.BIG_CASES))
def test_csg_larger_cases_against_oracle(name):
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    order, table = sp.csg_table(_dev(ptr), _dev(ind), is_symmetric=sym, **params)
    o_or, t_or = oracle.csg(ptr, ind, sym, with_table=True, **params)
    assert np.array_equal(table.cpu().numpy().view(np.uint64), t_or)
    assert np.array_equal(order.cpu().numpy(), o_or)


@pytest.mark.parametrize("name", ["hubsym", "rmat12", "m512", "bigchunk", "rmat16", "dense_ties",
                                  "dense_fill", "dense_m32", "dense_ragged", "dense_m96",
                                  "dense_m128", "dense_m128_ties", "zipf65k"])
def test_csg_against_reference_library(name):
    from oracle import ref
    if not ref.available():
        pytest.skip("reference build (oracle/_ref) not present")
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    dp, di = _dev(ptr), _dev(ind)
    prm = oracle.resolve_params(ptr.size - 1, ind.size, **params)
    order, table = sp.csg_table(dp, di, is_symmetric=sym, **params)
    r_order = ref.csg(dp, di, sym, **params)
    r_table = ref.csg_table(dp, di, sym, prm["k"], prm["oversampling"], prm["chunk_size"])
    assert torch.equal(table, r_table)
    assert torch.equal(order, r_order)


@pytest.mark.parametrize("name", ["band1000", "ragged", "hubsym", "zipf4k", "rmat12", "rmat16"])
@pytest.mark.parametrize("symmetric", [False, True])
def test_reorder_bit_exact(name, symmetric, golden):
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    order = oracle.csg(ptr, ind, sym, **params)
    rp, ri, rv = oracle.reorder(ptr, ind, order, val, symmetric=symmetric)
    gp, gi, gv = sp.reorder(_dev(ptr), _dev(ind), _dev(order), val=_dev(val), symmetric=symmetric)
    assert np.array_equal(gp.cpu().numpy(), rp)
    assert np.array_equal(gi.cpu().numpy(), ri)
    assert np.array_equal(gv.cpu().numpy(), rv)
    gp2, gi2 = sp.reorder(_dev(ptr), _dev(ind), _dev(order), symmetric=symmetric)
    assert np.array_equal(gi2.cpu().numpy(), ri) and np.array_equal(gp2.cpu().numpy(), rp)
    if symmetric and name in cases.CASES:
        assert np.array_equal(gp.cpu().numpy(), golden[name + "/sym_ptr"])
        assert np.array_equal(_sha(gi.cpu().numpy()), golden[name + "/sym_ind_sha256"])
        assert np.array_equal(_sha(gv.cpu().numpy()), golden[name + "/sym_val_sha256"])


def test_reorder_random_permutation_long_rows():
    # rows of every size class: <= 32 (warp), <= 2048 (shared memory), longer (global)
    sp = _sp()
    rng = np.random.default_rng(3)
    n = 6000
    lens = np.concatenate([rng.integers(0, 33, 5900), rng.integers(33, 2049, 90),
                           rng.integers(2049, 5000, 10)])
    rng.shuffle(lens)
    rows = np.repeat(np.arange(n), lens)
    cols = np.concatenate([rng.choice(n, l, replace=False) for l in lens])
    from chunkedgreedy_b200.synth import coo_to_csr
    ptr, ind, val = coo_to_csr(n, rows, cols, rng.standard_normal(rows.size))
    order = rng.permutation(n).astype(np.int32)
    for symmetric in (False, True):
        rp, ri, rv = oracle.reorder(ptr, ind, order, val, symmetric=symmetric)
        gp, gi, gv = sp.reorder(_dev(ptr), _dev(ind), _dev(order), val=_dev(val),
                                symmetric=symmetric)
        assert np.array_equal(gp.cpu().numpy(), rp)
        assert np.array_equal(gi.cpu().numpy(), ri)
        assert np.array_equal(gv.cpu().numpy(), rv)


def test_reorder_hub_row_of_120k_entries_under_a_global_permutation():
    # one row longer than any shared-memory sort can hold (the radix path, three digit
    # passes for 140,000 columns), under a permutation that moves columns across the whole
    # matrix, next to rows of every other size class
    sp = _sp()
    rng = np.random.default_rng(11)
    n = 140_000
    lens = rng.integers(0, 6, n)
    lens[5] = 120_000
    lens[77] = 4097
    lens[78] = 4096
    lens[79] = 33
    rows = np.repeat(np.arange(n), lens)
    cols = np.concatenate([rng.choice(n, l, replace=False) for l in lens])
    from chunkedgreedy_b200.synth import coo_to_csr
    ptr, ind, val = coo_to_csr(n, rows, cols, rng.standard_normal(rows.size))
    order = rng.permutation(n).astype(np.int32)
    for symmetric in (True, False):
        rp, ri, rv = oracle.reorder(ptr, ind, order, val, symmetric=symmetric)
        gp, gi, gv = sp.reorder(_dev(ptr), _dev(ind), _dev(order), val=_dev(val), symmetric=symmetric)
        assert np.array_equal(gp.cpu().numpy(), rp)
        assert np.array_equal(gi.cpu().numpy(), ri)
        assert np.array_equal(gv.cpu().numpy(), rv)
        gp2, gi2 = sp.reorder(_dev(ptr), _dev(ind), _dev(order), symmetric=symmetric)
        assert np.array_equal(gi2.cpu().numpy(), ri)


def test_reorder_round_trip_is_identity():
    sp = _sp()
    ptr, ind, val, sym, params = cases.build("rmat12")
    order = sp.chunk_similarity_greedy(_dev(ptr), _dev(ind))
    p1, i1, v1 = sp.reorder(_dev(ptr), _dev(ind), order, val=_dev(val), symmetric=True)
    inv = torch.empty_like(order)
    inv[order.long()] = torch.arange(order.numel(), dtype=torch.int32, device="cuda")
    p2, i2, v2 = sp.reorder(p1, i1, inv, val=v1, symmetric=True)
    assert np.array_equal(p2.cpu().numpy(), ptr) and np.array_equal(i2.cpu().numpy(), ind)
    assert np.array_equal(v2.cpu().numpy(), val)


@pytest.mark.parametrize("name", ["band1000", "zipf4k", "rmat12", "rmat16", "ragged"])
@pytest.mark.parametrize("w", [1, 7, 16, 32, 64, 128, 256])
def test_spmm_within_1e5_of_fp64(name, w):
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    n = ptr.size - 1
    B = np.random.default_rng(42).standard_normal((n, w)).astype(np.float32)
    C = sp.spmm(_dev(ptr), _dev(ind), _dev(val), _dev(B)).cpu().numpy()
    ref64, refabs = oracle.spmm_f64(ptr, ind, val, B)
    # tolerance stated by the workload definition: 1e-5 relative, scaled by sum |a*b|
    assert np.all(np.abs(C - ref64) <= 1e-5 * refabs + 1e-30)


SYMMETRIC_CASES = ["band1000", "hubsym", "stencil48", "stencil48_natural", "road3k", "rmat11gcn",
                   "stencil256", "rmat14gcn"]


@pytest.mark.parametrize("name", SYMMETRIC_CASES)
def test_symmetric_promise_reads_groups_off_the_csr_arrays_with_equal_results(name):
    # sporder/src/common/csr2csc.h:49-59: with is_symmetric the CSR arrays stand in for the
    # transpose.  Here that skips the chunk-local sort; table and permutation must not notice.
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    assert sym
    dp, di = _dev(ptr), _dev(ind)
    o1, t1 = sp.csg_table(dp, di, is_symmetric=True, **params)
    o0, t0 = sp.csg_table(dp, di, is_symmetric=False, **params)
    assert torch.equal(t1, t0) and torch.equal(o1, o0)
    i1, w1 = sp.similarity_graph(dp, di, is_symmetric=True)
    i0, w0 = sp.similarity_graph(dp, di, is_symmetric=False)
    assert torch.equal(i1, i0) and torch.equal(w1, w0)
    g1 = sp.chunk_greedy(dp, di, is_symmetric=True, chunk_size=256)
    g0 = sp.chunk_greedy(dp, di, is_symmetric=False, chunk_size=256)
    assert torch.equal(g1, g0)


@pytest.mark.parametrize("name", ["rmat12", "ragged", "m96", "chunk1", "dense_ragged"])
def test_a_false_symmetric_promise_still_gives_a_permutation(name):
    # like the reference, the library takes the promise at its word; on a pattern that is not
    # symmetric the candidates are then those of A + garbage, the result a valid permutation
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    assert not sym
    n = ptr.size - 1
    order = sp.chunk_similarity_greedy(_dev(ptr), _dev(ind), is_symmetric=True, **params)
    assert np.array_equal(np.sort(order.cpu().numpy()), np.arange(n, dtype=np.int32))
    chunk = params.get("chunk_size", 0) or 1024
    blocks = order.cpu().numpy() // chunk
    assert np.array_equal(blocks, np.arange(n) // chunk)  # rows never leave their chunk


def _rows_of_given_lengths(lengths, n_cols, seed):
    """CSR with the given row lengths, sorted distinct columns, N(0,1) values."""
    rng = np.random.default_rng(seed)
    ptr = np.zeros(len(lengths) + 1, dtype=np.int32)
    ptr[1:] = np.cumsum(lengths)
    ind = np.empty(ptr[-1], dtype=np.int32)
    for r, ln in enumerate(lengths):
        ind[ptr[r]:ptr[r + 1]] = np.sort(rng.choice(n_cols, size=ln, replace=False))
    val = rng.standard_normal(ptr[-1]).astype(np.float32)
    return ptr, ind, val


@pytest.mark.parametrize("w", [1, 2, 4, 8, 16, 32, 64, 96, 128, 256])
@pytest.mark.parametrize("longest", [16, 17, 40])
def test_spmm_on_units_of_short_rows(w, longest):
    # rows of 0..16 nonzeros go through the kernel's path for units of short rows, every
    # length and every remainder of a piece; with a few longer rows mixed in, units of both
    # kinds follow one another in the same launch
    sp = _sp()
    n = 6000
    rng = np.random.default_rng(7 + longest)
    lengths = rng.integers(0, 17, size=n)
    lengths[:40] = np.arange(40) % 17          # every length at the head of a unit
    if longest > 16:
        lengths[rng.choice(n, size=60, replace=False)] = longest
    ptr, ind, val = _rows_of_given_lengths(lengths, n, 11)
    B = np.random.default_rng(5).standard_normal((n, w)).astype(np.float32)
    C = sp.spmm(_dev(ptr), _dev(ind), _dev(val), _dev(B)).cpu().numpy()
    ref64, refabs = oracle.spmm_f64(ptr, ind, val, B)
    assert np.all(np.abs(C - ref64) <= 1e-5 * refabs + 1e-30)
    # and bit-equal run to run: no atomics on rows this short
    C2 = sp.spmm(_dev(ptr), _dev(ind), _dev(val), _dev(B)).cpu().numpy()
    assert np.array_equal(C, C2)


def test_spmm_is_linear_and_permutation_consistent():
    # size-independent properties at a larger size: A(x+y) = Ax + Ay, and
    # (P A P^T)(P x) = P (A x)
    sp = _sp()
    ptr, ind, val, sym, params = cases.build("rmat16")
    n = ptr.size - 1
    dp, di, dv = _dev(ptr), _dev(ind), _dev(val)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((n, 32), device="cuda", generator=g)
    y = torch.randn((n, 32), device="cuda", generator=g)
    ax, ay, axy = sp.spmm(dp, di, dv, x), sp.spmm(dp, di, dv, y), sp.spmm(dp, di, dv, x + y)
    scale = sp.spmm(dp, di, dv.abs(), x.abs() + y.abs())
    assert torch.all((axy - ax - ay).abs() <= 1e-5 * scale + 1e-30)
    order = sp.chunk_similarity_greedy(dp, di)
    p2, i2, v2 = sp.reorder(dp, di, order, val=dv, symmetric=True)
    lhs = sp.spmm(p2, i2, v2, x[order.long()])
    assert torch.all((lhs - ax[order.long()]).abs() <= 1e-5 * scale[order.long()] + 1e-30)


@pytest.mark.parametrize("name", ["rmat12", "hubsym", "ragged", "dense_ragged"])
def test_stats_and_timing_fields(name):
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    order, timing, stats = sp.chunk_similarity_greedy(_dev(ptr), _dev(ind), with_timing=True,
                                                      with_stats=True, is_symmetric=sym, **params)
    o_or, s_or = oracle.csg(ptr, ind, sym, with_stats=True, **params)
    assert np.array_equal(order.cpu().numpy(), o_or)
    assert set(timing) == {"wall_ms", "csr2csc_ms", "similarity_ms", "chunk_greedy_ms"}
    assert timing["wall_ms"] > 0
    for key in ("k_used", "m_used", "zero_degree_rows", "chunk_size_used", "chain_restarts"):
        assert stats[key] == s_or[key], key
    for key in ("avg_degree", "avg_edge_weight", "avg_followed_weight"):
        assert abs(stats[key] - s_or[key]) <= 1e-6 * max(1.0, abs(s_or[key])), key
    only_stats = sp.chunk_similarity_greedy(_dev(ptr), _dev(ind), with_stats=True, **params)
    assert isinstance(only_stats, tuple) and len(only_stats) == 2 and "k_used" in only_stats[1]


def test_errors_are_exceptions_and_context_survives():
    sp = _sp()
    ptr, ind, val, sym, params = cases.build("uniform")
    dp, di = _dev(ptr), _dev(ind)
    with pytest.raises(ValueError):
        sp.chunk_similarity_greedy(dp, di, k=200, oversampling=4.0)  # m = 800 > 512
    with pytest.raises(ValueError):
        sp.chunk_similarity_greedy(dp, di, oversampling=0.5)
    with pytest.raises(ValueError):
        sp.chunk_similarity_greedy(dp[:1], di)
    with pytest.raises(ValueError):
        sp.reorder(dp, di, dp[:5])
    with pytest.raises(ValueError):
        sp.chunk_similarity_greedy(dp.long(), di)
    order = sp.chunk_similarity_greedy(dp, di)  # still works after the failures
    assert np.array_equal(order.cpu().numpy(), oracle.csg(ptr, ind, sym))


def test_result_independent_of_repeat_and_context():
    sp = _sp()
    ptr, ind, val, sym, params = cases.build("rmat12")
    dp, di = _dev(ptr), _dev(ind)
    a = sp.chunk_similarity_greedy(dp, di)
    ctx = sp.Context()
    b = sp.chunk_similarity_greedy(dp, di, ctx=ctx)
    c = sp.chunk_similarity_greedy(dp, di, ctx=ctx)
    assert torch.equal(a, b) and torch.equal(b, c)
    ctx.close()


@pytest.mark.parametrize("name", ["band1000", "ragged", "hubsym", "rmat12", "rmat16", "dense_ragged",
                                  "tiny1"])
def test_pillar_count_matches_oracle_and_reference(name):
    from oracle import ref
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    n = ptr.size - 1
    d_ptr, d_ind = _dev(ptr), _dev(ind)
    for height in (1, 2, 16, 32, 33, 100, 1024, n + 5):
        want = oracle.count_pillars(ptr, ind, height)
        assert sp.count_pillars(d_ptr, d_ind, height) == want
        if ref.available() and height in (1, 16, 1024):
            assert ref.count_pillars(d_ptr, d_ind, height) == want
    assert sp.count_pillars(d_ptr, d_ind, 1) == ind.size  # sporder/tests/smoke.c:98-103
    with pytest.raises((ValueError, RuntimeError)):
        sp.count_pillars(d_ptr, d_ind, 0)


def test_pillar_count_of_the_reordered_matrix():
    # the metric is what the reorder is judged by: computed on P A P^T it must equal the
    # oracle's count on the oracle's reordered matrix
    sp = _sp()
    ptr, ind, val, sym, params = cases.build("hubsym")
    order = sp.chunk_similarity_greedy(_dev(ptr), _dev(ind), is_symmetric=True)
    p2, i2 = sp.reorder(_dev(ptr), _dev(ind), order, symmetric=True)
    rp, ri = oracle.reorder(ptr, ind, order.cpu().numpy(), symmetric=True)
    assert sp.count_pillars(p2, i2, 16) == oracle.count_pillars(rp, ri, 16)


@pytest.mark.parametrize("name", ["band1000", "ragged", "hubsym", "rmat12", "stencil48", "dense_ragged"])
def test_similarity_graph_matches_oracle_and_reference(name):
    from oracle import ref
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    d_ptr, d_ind = _dev(ptr), _dev(ind)
    for kw in (dict(), dict(k=8, oversampling=4.0), dict(k=40, oversampling=3.0)):
        idx, wgt, stats = sp.similarity_graph(d_ptr, d_ind, is_symmetric=sym, with_stats=True, **kw)
        o_idx, o_wgt = oracle.similarity_graph(ptr, ind, **kw)
        assert np.array_equal(idx.cpu().numpy(), o_idx)
        assert np.array_equal(wgt.cpu().numpy().view(np.uint32), o_wgt.view(np.uint32))
        assert stats["k_used"] == o_idx.shape[1]
        assert stats["zero_degree_rows"] == int((o_idx[:, 0] < 0).sum())
        assert abs(stats["avg_degree"] - (o_idx >= 0).sum() / o_idx.shape[0]) < 1e-9
        if ref.available():
            r_idx, r_wgt = ref.similarity_graph(d_ptr, d_ind, sym, **kw)
            assert np.array_equal(r_idx.cpu().numpy(), o_idx)
            assert np.array_equal(r_wgt.cpu().numpy().view(np.uint32), o_wgt.view(np.uint32))


@pytest.mark.parametrize("name", ["band1000", "ragged", "hubsym", "rmat12", "stencil48", "dense_ragged"])
def test_chunk_greedy_on_the_global_graph(name):
    from oracle import ref
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    d_ptr, d_ind = _dev(ptr), _dev(ind)
    for kw in (dict(), dict(k=8, oversampling=4.0, chunk_size=100), dict(chunk_size=4096)):
        order, stats = sp.chunk_greedy(d_ptr, d_ind, is_symmetric=sym, with_stats=True, **kw)
        o_order, o_st = oracle.chunk_greedy(ptr, ind, **kw)
        assert np.array_equal(order.cpu().numpy(), o_order)
        assert stats["k_used"] == o_st["k_used"]
        assert stats["chain_restarts"] == o_st["restarts"]
        # a diagnostic made of two fp32-accumulated sums (cg/stats_collector.cu:66-72)
        assert abs(stats["cut_weight_fraction"] - o_st["cut_weight_fraction"]) < 1e-5
        if ref.available():
            assert np.array_equal(ref.chunk_greedy(d_ptr, d_ind, sym, **kw).cpu().numpy(), o_order)


def test_harness_method_modules():
    # the shapes the reference's own scripts call: reorder_bench/methods/sporder_csg.py:25-70
    # and spmm_bench/base.py:8-65
    import scipy.sparse
    from chunkedgreedy_b200 import harness
    ptr, ind, val, sym, params = cases.build("hubsym")
    n = ptr.size - 1
    csr = scipy.sparse.csr_matrix((val, ind, ptr), shape=(n, n))
    res = harness.reorder(csr, {"k": 0, "oversampling": 0.0, "chunk_size": 0})
    assert res.effective_params["is_symmetric"] is False  # random values: A != A^T
    assert res.row_perm.dtype == np.int64
    assert np.array_equal(res.row_perm, oracle.csg(ptr, ind, False))
    assert res.reorder_time_ms > 0 and set(res.timing_breakdown) == {"csr2csc_ms", "similarity_ms",
                                                                     "chunk_greedy_ms"}
    pattern = scipy.sparse.csr_matrix((np.ones_like(val), ind, ptr), shape=(n, n))
    assert harness.reorder(pattern, {}).effective_params["is_symmetric"] is True
    m = harness.B200SpMM()
    m.build()
    prepared = m.prepare(csr)
    B = np.random.default_rng(3).standard_normal((n, 32)).astype(np.float32)
    C, kernel_ms = m.run(prepared, torch.from_numpy(B).cuda())
    c64, cabs = oracle.spmm_f64(ptr, ind, val, B)
    assert kernel_ms > 0
    assert np.all(np.abs(C.cpu().numpy() - c64) <= 1e-5 * cabs + 1e-30)


def test_host_entry_point_matches_device_path():
    sp = _sp()
    ptr, ind, val, sym, params = cases.build("rmat12")
    hp, hi = torch.from_numpy(ptr).pin_memory(), torch.from_numpy(ind).pin_memory()
    out = sp.chunk_similarity_greedy_host(hp, hi)
    assert np.array_equal(out.numpy(), oracle.csg(ptr, ind, sym))


def test_native_library_is_the_one_that_ran():
    sp = _sp()
    before = sp.kernel_launches()
    ptr, ind, val, sym, params = cases.build("uniform")
    sp.chunk_similarity_greedy(_dev(ptr), _dev(ind))
    assert sp.kernel_launches() >= before + 5
    maps = open("/proc/self/maps").read()
    assert "libsporder_b200.so" in maps


def test_gcn_gradients_match_dense_reference_and_reordering_is_equivalent():
    # the SpMM autograd function against a dense torch fp32 reference of the same op,
    # and training on P A P^T with permuted features gives the same losses
    sp = _sp()
    from chunkedgreedy_b200 import gcn
    ptr, ind, val, sym, params = cases.build("rmat11gcn")
    n = ptr.size - 1
    dp, di, dv = _dev(ptr), _dev(ind), _dev(val)
    dense = torch.zeros((n, n), device="cuda")
    rows = torch.repeat_interleave(torch.arange(n, device="cuda"), (dp[1:] - dp[:-1]).long())
    dense[rows, di.long()] = dv
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((n, 32), device="cuda", generator=g, requires_grad=True)
    op = gcn.GraphOperator(dp, di, dv)
    y = gcn.SpMMFn.apply(x, op)
    y.square().sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    yr = dense @ xr
    yr.square().sum().backward()
    assert torch.allclose(y, yr, rtol=1e-4, atol=1e-5)
    assert torch.allclose(x.grad, xr.grad, rtol=1e-4, atol=1e-4)
    feats = torch.randn((n, 16), device="cuda", generator=g)
    labels = torch.randint(0, 4, (n,), device="cuda", generator=g)
    res = gcn.reorder_and_train(dp, di, dv, feats, labels, hidden=16, classes=4, epochs=5,
                                warmup=0)
    a, b = res["original"]["final_loss"], res["reordered"]["final_loss"]
    assert abs(a - b) <= 1e-3 * max(1.0, abs(a))
    assert sorted(res["order"].cpu().tolist()) == list(range(n))


@pytest.mark.parametrize("name", ["stencil1024", "road2m"])
def test_full_size_streaming_workloads_bit_exact(name):
    # benchmark configurations 2 and 3 at their full sizes (1.05 M / 2 M rows): the oracle
    # finishes in seconds because relabelled meshes have almost no in-chunk candidates
    sp = _sp()
    from chunkedgreedy_b200 import synth
    w = synth.make_workload(name)
    order, table = sp.csg_table(_dev(w["ptr"]), _dev(w["ind"]), is_symmetric=True)
    o_or, t_or = oracle.csg(w["ptr"], w["ind"], True, with_table=True)
    assert np.array_equal(order.cpu().numpy(), o_or)
    assert np.array_equal(table.cpu().numpy().view(np.uint64), t_or)


def test_full_size_power_law_workload_properties():
    # benchmark configuration 4 at scale 20 against the oracle, bit-exact, and the structural
    # invariants of the reference's smoke test on the result (valid permutation, every chunk a
    # permutation of its own rows that starts at the chunk's first row), plus the
    # P A P^T round trip
    sp = _sp()
    from chunkedgreedy_b200 import synth
    ptr, ind, val = synth.rmat(scale=20, seed=3)
    n = ptr.size - 1
    dp, di, dv = _dev(ptr), _dev(ind), _dev(val)
    order = sp.chunk_similarity_greedy(dp, di)
    assert np.array_equal(order.cpu().numpy(), oracle.csg(ptr, ind, False))
    o = order.cpu().numpy().reshape(-1, 1024)
    assert np.array_equal(o[:, 0], np.arange(0, n, 1024))
    assert np.array_equal(np.sort(o, axis=1), np.arange(n).reshape(-1, 1024))
    p2, i2, v2 = sp.reorder(dp, di, order, val=dv, symmetric=True)
    inv = torch.empty_like(order)
    inv[order.long()] = torch.arange(n, dtype=torch.int32, device="cuda")
    p3, i3, v3 = sp.reorder(p2, i2, inv, val=v2, symmetric=True)
    assert torch.equal(p3, dp) and torch.equal(i3, di) and torch.equal(v3, dv)



def test_full_size_gcn_workload_bit_exact():
    # benchmark configuration 5 at full size: R-MAT scale 20 symmetrised with self loops,
    # k = nnz / n = 30, 128 slots (four cells per lane, the widest sketch resolved in rounds)
    sp = _sp()
    from chunkedgreedy_b200 import synth
    w = synth.make_workload("rmat20gcn")
    order = sp.chunk_similarity_greedy(_dev(w["ptr"]), _dev(w["ind"]), is_symmetric=True)
    assert np.array_equal(order.cpu().numpy(), oracle.csg(w["ptr"], w["ind"], True))


def test_heavy_rows_that_do_not_fit_the_stream_buffer_take_the_light_path():
    # The heaviest rows are computed from a materialised copy of their candidate stream; rows
    # whose copy does not fit the buffer go through the kernel of the lighter rows instead.
    # A context limited to 100,000 stream elements keeps one row of this case (89,700
    # candidates each) on the fast path and sends 299 back; no limit keeps all 300.
    sp = _sp()
    from chunkedgreedy_b200 import _lib
    lib = _lib.load()
    for name, limit in (("dense_ties", 100_000), ("dense_ragged", 150_000), ("dense_m128", 70_000),
                        ("dense_ties", 1000)):
        ptr, ind, val, sym, params = cases.build(name)
        o_or, t_or = oracle.csg(ptr, ind, sym, with_table=True, **params)
        ctx = sp.Context()
        lib.sporder_context_set_stream_limit(ctx.handle, limit)
        for _ in range(2):  # the second call plans from what the first one reported
            order, table = sp.csg_table(_dev(ptr), _dev(ind), ctx=ctx, **params)
            assert np.array_equal(table.cpu().numpy().view(np.uint64), t_or), (name, limit)
            assert np.array_equal(order.cpu().numpy(), o_or), (name, limit)
        lib.sporder_context_set_stream_limit(ctx.handle, 0)
        order, table = sp.csg_table(_dev(ptr), _dev(ind), ctx=ctx, **params)
        assert np.array_equal(table.cpu().numpy().view(np.uint64), t_or)
        ctx.close()


AHEAD_CASES = ["rmat12", "hubsym", "ragged", "m96", "m512", "bigchunk", "dense_ties", "dense_fill",
               "dense_ragged", "dense_c4096", "dense_m128", "dense_m256", "rmat16"]


@pytest.mark.parametrize("name", AHEAD_CASES)
def test_running_one_chunk_ahead_changes_nothing(name):
    # Large calls transpose the chunk with the most nonzeros first and start the chains of
    # its heaviest rows on a second stream while the rest is transposed.  With the threshold
    # at one nonzero every call of two chunks takes that route, whatever its size: same table,
    # same permutation as the CPU restatement, on a first call (stream buffer cut in halves)
    # and on later ones (cut by what each part asked for); and the same with the route closed.
    sp = _sp()
    ptr, ind, val, sym, params = cases.build(name)
    o_or, t_or = oracle.csg(ptr, ind, False, with_table=True, **params)
    ctx = sp.Context()
    ctx.set_ahead_threshold(1)
    for _ in range(3):
        order, table = sp.csg_table(_dev(ptr), _dev(ind), ctx=ctx, **params)
        assert np.array_equal(table.cpu().numpy().view(np.uint64), t_or), name
        assert np.array_equal(order.cpu().numpy(), o_or), name
    ctx.set_stream_limit(200_000)  # ... and with both parts short of room for their streams
    order, table = sp.csg_table(_dev(ptr), _dev(ind), ctx=ctx, **params)
    assert np.array_equal(table.cpu().numpy().view(np.uint64), t_or), name
    ctx.set_stream_limit(0)
    ctx.set_ahead_threshold(-1)
    order, table = sp.csg_table(_dev(ptr), _dev(ind), ctx=ctx, **params)
    assert np.array_equal(table.cpu().numpy().view(np.uint64), t_or), name
    assert np.array_equal(order.cpu().numpy(), o_or), name
    ctx.close()


def test_running_one_chunk_ahead_at_scale_20_and_with_statistics():
    # R-MAT scale 20 (15.5 M nonzeros, 1024 chunks): chunk 0 holds the rows with the longest
    # streams, which is the case the route is made for
    sp = _sp()
    from chunkedgreedy_b200 import synth
    ptr, ind, val = synth.rmat(scale=20, edge_factor=16, seed=3)
    dp, di = _dev(ptr), _dev(ind)
    plain = sp.Context()
    plain.set_ahead_threshold(-1)
    o0, t0 = sp.csg_table(dp, di, ctx=plain)
    ahead = sp.Context()
    ahead.set_ahead_threshold(1)
    for _ in range(2):
        o1, t1 = sp.csg_table(dp, di, ctx=ahead)
        assert torch.equal(t1, t0) and torch.equal(o1, o0)
    o2, tm, st = sp.chunk_similarity_greedy(dp, di, ctx=ahead, with_timing=True, with_stats=True)
    _, _, st0 = sp.chunk_similarity_greedy(dp, di, ctx=plain, with_timing=True, with_stats=True)
    assert torch.equal(o2, o0) and st == st0 and tm["wall_ms"] > 0
    plain.close()
    ahead.close()


def test_workspace_is_in_proportion_to_the_input():
    # a small matrix must not make the context hold the gigabyte a large one needs
    sp = _sp()
    ptr, ind, val, sym, params = cases.build("rmat12")
    ctx = sp.Context()
    sp.chunk_similarity_greedy(_dev(ptr), _dev(ind), ctx=ctx)
    assert ctx.workspace_bytes() < 64 << 20
    sp.count_pillars(_dev(ptr), _dev(ind), 64, ctx=ctx)
    assert ctx.workspace_bytes() < 64 << 20
    ctx.close()


def test_shard_must_hold_whole_chunks():
    sp = _sp()
    from chunkedgreedy_b200 import dist as csgdist
    ptr, ind, val, sym, params = cases.build("rmat12")
    n = ptr.size - 1
    pl, il = csgdist.extract_shard(ptr, ind, 1000, 2024)  # starts in the middle of a chunk
    with pytest.raises(RuntimeError, match="multiple of the chunk size"):
        csgdist.csg_shard(_dev(pl), _dev(il), n, 1000, k=16, chunk_size=1024)
    pl, il = csgdist.extract_shard(ptr, ind, 3072, n)
    with pytest.raises(RuntimeError, match="does not lie inside"):
        csgdist.csg_shard(_dev(pl), _dev(il), n - 1, 3072, k=16, chunk_size=1024)
    order = csgdist.csg_shard(_dev(pl), _dev(il), n, 3072, k=16, chunk_size=1024)
    assert np.array_equal(order.cpu().numpy(), oracle.csg(ptr, ind, False)[3072:])


@pytest.mark.parametrize("name", ["rmat16", "dense_ragged", "bigchunk"])
def test_row_shards_that_run_one_chunk_ahead(name):
    # the shards of a multi-GPU run, one after the other on this GPU, each forced onto the
    # route that runs its heaviest chunk ahead: together they are the single-GPU permutation
    sp = _sp()
    from chunkedgreedy_b200 import dist as csgdist
    ptr, ind, val, sym, params = cases.build(name)
    n = ptr.size - 1
    chunk = params.get("chunk_size", 0) or 1024
    k = params.get("k", 0) or csgdist.resolve_k(n, ind.size, 0)
    want = oracle.csg(ptr, ind, False, **params)
    ctx = sp.Context()
    ctx.set_ahead_threshold(1)
    parts = []
    for r0, r1 in csgdist.shard_bounds(ptr, chunk, 3):
        pl, il = csgdist.extract_shard(ptr, ind, r0, r1)
        kw = {key: v for key, v in params.items() if key not in ("k", "chunk_size")}
        parts.append(csgdist.csg_shard(_dev(pl), _dev(il), n, r0, k=k, chunk_size=chunk, ctx=ctx, **kw).cpu().numpy())
    assert np.array_equal(np.concatenate(parts), want)
    ctx.close()


def test_spmm_of_a_row_block_against_the_whole_product():
    # the row-partitioned product: a block of rows times the whole dense operand
    sp = _sp()
    from chunkedgreedy_b200 import dist as csgdist
    ptr, ind, val, sym, params = cases.build("rmat16")
    n = ptr.size - 1
    dp, di, dv = _dev(ptr), _dev(ind), _dev(val)
    B = torch.randn((n, 32), device="cuda")
    whole = sp.spmm(dp, di, dv, B)
    scale = sp.spmm(dp, di, dv.abs(), B.abs())
    bounds = csgdist.spmm_row_bounds(dp, 3)
    assert bounds[0][0] == 0 and bounds[-1][1] == n
    for r0, r1 in bounds:
        pl, il, vl = csgdist.spmm_shard(dp, di, dv, r0, r1)
        part = sp.spmm(pl, il, vl, B, n_cols=n)
        # (not bitwise: the pieces of a long row are added in whatever order they finish)
        assert torch.all((part - whole[r0:r1]).abs() <= 1e-5 * scale[r0:r1] + 1e-30)
    with pytest.raises(ValueError):
        sp.spmm(pl, il, vl, B)  # without n_cols the operand must be square with the block


def test_results_come_back_in_the_callers_array_framework():
    # sporder/python/sporder/__init__.py:28-39: arrays of another framework go in through
    # DLPack and results come back through that framework's from_dlpack
    import sys
    import types
    sp = _sp()

    class Foreign:
        def __init__(self, t):
            self.t = t

        def __dlpack__(self, stream=None):
            return self.t.__dlpack__()

        def __dlpack_device__(self):
            return self.t.__dlpack_device__()

    mod = types.ModuleType("foreignxp")
    mod.from_dlpack = lambda t: Foreign(torch.from_dlpack(t))
    sys.modules["foreignxp"] = mod
    Foreign.__module__ = "foreignxp.core"
    try:
        ptr, ind, val, sym, params = cases.build("rmat12")
        order = sp.chunk_similarity_greedy(Foreign(_dev(ptr)), Foreign(_dev(ind)))
        assert isinstance(order, Foreign)
        assert np.array_equal(order.t.cpu().numpy(), oracle.csg(ptr, ind, False))
        out = sp.reorder(Foreign(_dev(ptr)), _dev(ind), order, symmetric=True)
        assert all(isinstance(a, Foreign) for a in out)
        assert isinstance(sp.chunk_similarity_greedy(_dev(ptr), _dev(ind)), torch.Tensor)
    finally:
        del sys.modules["foreignxp"]


def test_default_context_follows_the_arrays_device():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sp = _sp()
    ptr, ind, val, sym, params = cases.build("rmat12")
    with torch.cuda.device(0):
        dp, di = (torch.from_numpy(a).to("cuda:1") for a in (ptr, ind))
        order = sp.chunk_similarity_greedy(dp, di)  # device 0 is current, the arrays live on 1
        assert order.device.index == 1 and torch.cuda.current_device() == 0
        assert np.array_equal(order.cpu().numpy(), oracle.csg(ptr, ind, False))


def _nccl_worker(rank, world, port, result_path):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    from chunkedgreedy_b200 import dist as csgdist
    ptr, ind, val, sym, params = cases.build("rmat16")
    order = csgdist.chunk_similarity_greedy_sharded(ptr, ind, **params)
    # the SpMM the reorder feeds, row-partitioned: every rank its rows, gathered for the check
    import chunkedgreedy_b200 as sp
    dp, di, dv = _dev(ptr), _dev(ind), _dev(val)
    p2, i2, v2 = sp.reorder(dp, di, order, val=dv, symmetric=True)
    B = torch.from_numpy(np.random.default_rng(9).standard_normal((ptr.size - 1, 32)).astype(np.float32)).cuda()
    c = csgdist.spmm_sharded(p2, i2, v2, B, gather=True)
    if rank == 0:
        np.save(result_path, order.cpu().numpy())
        np.save(result_path + ".c.npy", c.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_row_shards_equal_single_gpu(tmp_path):
    # needs two GPUs; the host-side sharding logic itself is covered on CPU (gloo)
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    path = str(tmp_path / "order.npy")
    mp.spawn(_nccl_worker, args=(2, port, path), nprocs=2, join=True)
    ptr, ind, val, sym, params = cases.build("rmat16")
    want = oracle.csg(ptr, ind, False, **params)
    assert np.array_equal(np.load(path), want)
    rp, ri, rv = oracle.reorder(ptr, ind, want, val, symmetric=True)
    B = np.random.default_rng(9).standard_normal((ptr.size - 1, 32)).astype(np.float32)
    c64, cabs = oracle.spmm_f64(rp, ri, rv, B)
    assert np.all(np.abs(np.load(path + ".c.npy") - c64) <= 1e-5 * cabs + 1e-30)
