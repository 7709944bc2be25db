"""Pins the CPU oracle against outputs of the reference library itself.

tests/golden/csg_golden.npz was recorded on a B200 from the unmodified reference
sources (see tests/golden/make_golden.py).  Bit-exact: permutations, top-k tables
(full arrays for small cases, SHA-256 otherwise) and the symmetric reorder.
"""
import hashlib

import numpy as np
import pytest

import cases
import oracle


def _sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8)


@pytest.mark.parametrize("name", list(cases.CASES))
def test_oracle_matches_reference_outputs(name, golden):
    ptr, ind, val, sym, params = cases.build(name)
    order, table = oracle.csg(ptr, ind, sym, with_table=True, **params)
    n, nnz, k, M, chunk = golden[name + "/shape"]
    prm = oracle.resolve_params(ptr.size - 1, ind.size, **params)
    assert (n, nnz, k, M, chunk) == (ptr.size - 1, ind.size, prm["k"], prm["M"], prm["chunk_size"])
    assert np.array_equal(order, golden[name + "/order"])
    assert np.array_equal(_sha(table), golden[name + "/table_sha256"])
    if name + "/table" in golden:
        assert np.array_equal(table, golden[name + "/table"])
    rp, ri, rv = oracle.reorder(ptr, ind, order, val, symmetric=True)
    assert np.array_equal(rp, golden[name + "/sym_ptr"])
    assert np.array_equal(_sha(ri), golden[name + "/sym_ind_sha256"])
    assert np.array_equal(_sha(rv), golden[name + "/sym_val_sha256"])


def test_band_fixture_invariants():
    # checks of the reference's C smoke test (sporder/tests/smoke.c:88-115) on its fixture
    ptr, ind, val, sym, params = cases.build("band1000")
    order, table = oracle.csg(ptr, ind, sym, with_table=True)
    assert sorted(order.tolist()) == list(range(1000))
    idx, w = oracle.decode_table(table)
    assert 0 < idx[0, 0] < 1000
    rp, ri = oracle.reorder(ptr, ind, order)
    assert rp[-1] == ind.size


@pytest.mark.parametrize("name", ["hub_c700", "rmat12", "ragged", "chunk1"])
def test_structural_invariants(name):
    ptr, ind, val, sym, params = cases.build(name)
    n = ptr.size - 1
    order = oracle.csg(ptr, ind, sym, **params)
    chunk = oracle.resolve_params(n, ind.size, **params)["chunk_size"]
    assert sorted(order.tolist()) == list(range(n))
    for s in range(0, n, chunk):
        e = min(s + chunk, n)
        seg = order[s:e]
        assert seg[0] == s  # the chain starts at the chunk's first row
        assert seg.min() == s and seg.max() == e - 1 and len(set(seg.tolist())) == e - s


def test_thread_count_does_not_change_bits():
    ptr, ind, val, sym, params = cases.build("rmat12")
    old = oracle.num_threads()
    oracle.set_num_threads(1)
    a = oracle.csg(ptr, ind, sym, with_table=True, **params)
    oracle.set_num_threads(max(2, old))
    b = oracle.csg(ptr, ind, sym, with_table=True, **params)
    oracle.set_num_threads(old)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_chunk_covering_matrix_equals_any_larger_chunk():
    ptr, ind, val, sym, params = cases.build("onechunk")
    n = ptr.size - 1
    a = oracle.csg(ptr, ind, sym, chunk_size=n)
    b = oracle.csg(ptr, ind, sym, chunk_size=4 * n)
    assert np.array_equal(a, b)


def test_parameter_resolution():
    # sporder/src/sporder.cpp:147-155 and chunk_similarity_top_k.cu:143-147
    assert oracle.resolve_params(1000, 5000)["k"] == 16
    assert oracle.resolve_params(1000, 40000)["k"] == 40
    assert oracle.resolve_params(1000, 400000, oversampling=1.5)["k"] == 256
    p = oracle.resolve_params(1000, 100000)
    assert (p["k"], p["M"], p["chunk_size"], p["oversampling"]) == (100, 416, 1024, 4.0)
    with pytest.raises(ValueError):
        oracle.resolve_params(1000, 200000)  # k = 200 -> m = 800 > 512
    with pytest.raises(ValueError):
        oracle.resolve_params(1000, 5000, oversampling=0.5)
    p = oracle.resolve_params(10, 10, k=24, oversampling=3.5)
    assert (p["m_used"], p["M"]) == (96, 96)


def test_reorder_rows_and_symmetric_small():
    ptr = np.array([0, 2, 3, 5], dtype=np.int32)
    ind = np.array([0, 2, 1, 0, 1], dtype=np.int32)
    val = np.array([1, 2, 3, 4, 5], dtype=np.float32)
    order = np.array([2, 0, 1], dtype=np.int32)
    rp, ri, rv = oracle.reorder(ptr, ind, order, val, symmetric=False)
    assert rp.tolist() == [0, 2, 4, 5] and ri.tolist() == [0, 1, 0, 2, 1]
    assert rv.tolist() == [4, 5, 1, 2, 3]
    rp, ri, rv = oracle.reorder(ptr, ind, order, val, symmetric=True)
    # old2new = [1, 2, 0]; row 0 <- old 2 {0,1}->{1,2}; row 1 <- old 0 {0,2}->{1,0}; row 2 <- old 1
    assert ri.tolist() == [1, 2, 0, 1, 2] and rv.tolist() == [4, 5, 2, 1, 3]


def test_spmm_oracles_agree():
    ptr, ind, val, sym, params = cases.build("zipf4k")
    B = np.random.default_rng(0).standard_normal((ptr.size - 1, 8)).astype(np.float32)
    c64, cabs = oracle.spmm_f64(ptr, ind, val, B)
    c32 = oracle.spmm_f32(ptr, ind, val, B)
    assert np.all(np.abs(c32 - c64) <= 1e-5 * cabs + 1e-30)


@pytest.mark.parametrize("name", ["band1000", "ragged", "hubsym", "rmat12", "stencil48"])
def test_oracle_pillar_count_against_brute_force(name):
    # sporder/src/count_pillars.cu:38-85 counts distinct (row // height, column) keys
    ptr, ind, val, sym, params = cases.build(name)
    n = ptr.size - 1
    rows = np.repeat(np.arange(n, dtype=np.int64), np.diff(ptr))
    for height in (1, 2, 16, 33, 1000, n + 5):
        brute = np.unique((rows // height) * n + ind).size
        assert oracle.count_pillars(ptr, ind, height) == brute
    # the reference's smoke test: one window per row counts every nonzero
    # (sporder/tests/smoke.c:98-103)
    assert oracle.count_pillars(ptr, ind, 1) == ind.size


def test_oracle_pillar_count_matches_reference_outputs():
    # tests/golden/pillars_golden.json: sporder_count_pillars of the reference library on a
    # B200 (tests/golden/make_pillars_golden.py)
    import json
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pillars_golden.json")
    recorded = json.load(open(path))
    assert sorted(recorded) == sorted(cases.CASES)
    for name, by_height in recorded.items():
        ptr, ind, val, sym, params = cases.build(name)
        for height, want in by_height.items():
            assert oracle.count_pillars(ptr, ind, int(height)) == want, (name, height)
