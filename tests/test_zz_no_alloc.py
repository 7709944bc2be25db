"""The allocation-free SpMM entry point (sporder_spmm_static) against sporder_spmm.

Some hosts of the library cannot let it call cudaMalloc: the application owns all device
memory through its own pool, or driver allocations are banned on the request path because
they stall the device.  For them the SpMM keeps its only scratch (the queue of long rows)
in a fixed array inside the library.  That array is shared by all calls and keeps the
previous call's contents, so the test calls twice in a row: the second call must not be
confused by what the first one left behind.  The file name sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _matrix_with_long_rows(seed):
    from chunkedgreedy_b200.synth import coo_to_csr
    rng = np.random.default_rng(seed)
    n = 5000
    lens = rng.integers(0, 40, n)
    lens[rng.choice(n, 12, replace=False)] = rng.integers(1100, 4500, 12)  # rows past the split
    rows = np.repeat(np.arange(n), lens)
    cols = np.concatenate([rng.choice(n, l, replace=False) for l in lens])
    return coo_to_csr(n, rows, cols, rng.standard_normal(rows.size))


@pytest.mark.parametrize("w", [32, 128, 7])
def test_static_scratch_spmm_matches_spmm_twice_in_a_row(w):
    import chunkedgreedy_b200 as sp
    import oracle
    from chunkedgreedy_b200 import _lib
    lib = _lib.load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream or 1)
    for seed in (1, 2):  # two calls in a row, different matrices: the queue is reused
        ptr, ind, val = _matrix_with_long_rows(seed)
        n, nnz = ptr.size - 1, ind.size
        dp, di, dv = (torch.from_numpy(a).cuda() for a in (ptr, ind, val))
        B = torch.randn((n, w), device="cuda")
        want = sp.spmm(dp, di, dv, B)
        scale = sp.spmm(dp, di, dv.abs(), B.abs())
        got = torch.full((n, w), float("nan"), device="cuda")
        rc = lib.sporder_spmm_static(n, nnz, w, dp.data_ptr(), di.data_ptr(), dv.data_ptr(),
                                     B.data_ptr(), got.data_ptr(), stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        # same tolerance as the other SpMM tests: 1e-5, scaled by sum |a*b|
        assert torch.all((got - want).abs() <= 1e-5 * scale + 1e-30)
        # and directly against the fp64 product of the CPU checker
        c64, cabs = oracle.spmm_f64(ptr, ind, val, B.cpu().numpy())
        assert np.all(np.abs(got.cpu().numpy() - c64) <= 1e-5 * cabs + 1e-30)


def test_static_scratch_spmm_allocates_nothing_and_takes_the_default_stream():
    # what the entry point is for: after its one-time set-up a call must leave the amount of
    # free device memory and the workspace of every context exactly as it found them
    import chunkedgreedy_b200 as sp
    from chunkedgreedy_b200 import _lib
    lib = _lib.load()
    ptr, ind, val = _matrix_with_long_rows(3)
    n, nnz, w = ptr.size - 1, ind.size, 32
    dp, di, dv = (torch.from_numpy(a).cuda() for a in (ptr, ind, val))
    B = torch.randn((n, w), device="cuda")
    ctx = sp.Context()
    want = sp.spmm(dp, di, dv, B, ctx=ctx)
    scale = sp.spmm(dp, di, dv.abs(), B.abs(), ctx=ctx)
    got = torch.empty((n, w), device="cuda")

    def call(stream):
        rc = lib.sporder_spmm_static(n, nnz, w, dp.data_ptr(), di.data_ptr(), dv.data_ptr(),
                                     B.data_ptr(), got.data_ptr(), stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()

    call(None)  # warm: the address look-up of the first call on this device is done
    free_before, _ = torch.cuda.mem_get_info()
    ws_before = ctx.workspace_bytes()
    got.fill_(float("nan"))
    call(None)  # NULL names the default stream
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert ctx.workspace_bytes() == ws_before
    assert torch.all((got - want).abs() <= 1e-5 * scale + 1e-30)
    ctx.close()


def test_static_scratch_spmm_rejects_sizes_beyond_its_array():
    from chunkedgreedy_b200 import _lib
    lib = _lib.load()
    d = torch.zeros(4, dtype=torch.int32, device="cuda")
    f = torch.zeros(4, dtype=torch.float32, device="cuda")
    rc = lib.sporder_spmm_static(2, 65536 * 1024, 1, d.data_ptr(), d.data_ptr(), f.data_ptr(),
                                 f.data_ptr(), f.data_ptr(), None)
    assert rc == -1 and "exceeds the fixed scratch" in _lib.last_error()
