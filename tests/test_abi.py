"""The C-ABI library loads and exports every symbol include/sporder_b200.h declares.
No compute calls: this runs without a GPU."""
import ctypes
import os
import re

from chunkedgreedy_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sporder_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sporder_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported(built_lib):
    lib = ctypes.CDLL(built_lib)
    declared = _declared_symbols()
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(lib, name), name


def test_binding_table_covers_header(built_lib):
    assert sorted(_lib.SYMBOLS) == _declared_symbols()
    _lib.load()


def test_struct_layouts_match_reference_header():
    # sporder/include/sporder.h:203-222: timing = double + 3 floats, stats = 48 bytes
    assert ctypes.sizeof(_lib.CsgTiming) == 24
    assert ctypes.sizeof(_lib.CsgStats) == 48
    assert _lib.CsgStats.avg_degree.offset == 8
    assert _lib.CsgStats.zero_degree_rows.offset == 24
    assert _lib.CsgStats.avg_followed_weight.offset == 40


def test_null_context_is_an_error_not_a_crash(built_lib):
    lib = _lib.load()
    lib.sporder_chunk_similarity_greedy(None, 1, 0, None, None, False, 0, 0.0, 0, None, None, None)
    assert _lib.last_error() == "null context"
    assert lib.sporder_spmm(None, 1, 0, 1, None, None, None, None, None) == -1


def test_no_cpu_fallback_message(monkeypatch):
    import chunkedgreedy_b200 as sp
    import torch
    if torch.cuda.is_available():
        return
    try:
        sp.Context()
    except RuntimeError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("Context() must fail without a CUDA device")


def test_harness_module_imports_without_gpu_or_harness():
    from chunkedgreedy_b200 import harness
    assert harness.B200SpMM().name == "sporder-b200-spmm"
    r = harness.ReorderResult(row_perm=None, reorder_time_ms=1.0)
    assert r.prep_time_ms == 0.0 and r.timing_breakdown == {}


def test_amortization_and_breakeven_formulas():
    # bench/spmm/scripts/compute_amortization.py:63-66 and analysis/e2e.py:32-33
    from chunkedgreedy_b200 import harness
    assert harness.amortization_runs(40.0, 2.5, 2.0) == 80.0
    assert harness.amortization_runs(40.0, 2.0, 2.0) == float("inf")
    assert harness.amortization_runs(40.0, 2.0, 2.5) == float("inf")
    assert harness.format_amortization(float("inf")) == "inf"
    assert harness.format_amortization(80.0) == "80"
    import importlib.util
    if importlib.util.find_spec("torch") is None:
        return
    from chunkedgreedy_b200 import gcn
    assert gcn.breakeven_epochs(60.0, 1.5, 13.0, 12.5) == 123.0
    assert gcn.breakeven_epochs(60.0, 1.5, 12.5, 12.5) == float("inf")


def test_library_path_can_name_another_build(monkeypatch):
    # the checked build is loaded through SPORDER_B200_LIBRARY
    import importlib
    monkeypatch.setenv("SPORDER_B200_LIBRARY", "/nowhere/libsporder_b200_checked.so")
    mod = importlib.reload(_lib)
    try:
        assert mod.LIB_PATH == "/nowhere/libsporder_b200_checked.so"
        try:
            mod.load()
        except RuntimeError as e:
            assert "missing" in str(e)
        else:
            raise AssertionError("a missing library must fail loudly")
    finally:
        monkeypatch.delenv("SPORDER_B200_LIBRARY")
        importlib.reload(_lib)
