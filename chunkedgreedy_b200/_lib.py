"""ctypes binding of libsporder_b200.so (include/sporder_b200.h).

There is no fallback: if the CUDA library is missing or fails to load, importing
the package's compute entry points raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# SPORDER_B200_LIBRARY names another build of the same library (the checked build)
LIB_PATH = os.environ.get("SPORDER_B200_LIBRARY") or os.path.join(HERE, "libsporder_b200.so")

_lib = None


class CsgTiming(C.Structure):
    _fields_ = [("wall_ms", C.c_double), ("csr2csc_ms", C.c_float),
                ("similarity_ms", C.c_float), ("chunk_greedy_ms", C.c_float)]


class CsgStats(C.Structure):
    _fields_ = [("k_used", C.c_int32), ("m_used", C.c_int32), ("avg_degree", C.c_double),
                ("avg_edge_weight", C.c_double), ("zero_degree_rows", C.c_int32),
                ("chunk_size_used", C.c_int32), ("chain_restarts", C.c_int32),
                ("avg_followed_weight", C.c_double)]


# every symbol include/sporder_b200.h declares: name -> (restype, argtypes)
_P = C.c_void_p
class CgStats(C.Structure):
    _fields_ = [("k_used", C.c_int32), ("m_used", C.c_int32), ("avg_degree", C.c_double),
                ("avg_edge_weight", C.c_double), ("zero_degree_rows", C.c_int32),
                ("chunk_size_used", C.c_int32), ("chain_restarts", C.c_int32),
                ("avg_followed_weight", C.c_double), ("cut_weight_fraction", C.c_double)]


class SimTiming(C.Structure):
    _fields_ = [("wall_ms", C.c_double), ("csr2csc_ms", C.c_float), ("similarity_ms", C.c_float),
                ("unpack_ms", C.c_float)]


class SimStats(C.Structure):
    _fields_ = [("k_used", C.c_int32), ("m_used", C.c_int32), ("avg_degree", C.c_double),
                ("avg_edge_weight", C.c_double), ("zero_degree_rows", C.c_int32)]


SYMBOLS = {
    "sporder_context_create": (_P, []),
    "sporder_context_destroy": (None, [_P]),
    "sporder_chunk_similarity_greedy": (None, [_P, C.c_int32, C.c_int32, _P, _P, C.c_bool,
                                               C.c_int32, C.c_float, C.c_int32, _P,
                                               C.POINTER(CsgTiming), C.POINTER(CsgStats)]),
    "sporder_reorder": (None, [_P, C.c_int32, C.c_int32, _P, _P, _P, _P, C.c_int, _P, _P, _P]),
    "sporder_last_error": (C.c_char_p, []),
    "sporder_context_set_stream": (None, [_P, _P]),
    "sporder_context_workspace_bytes": (C.c_uint64, [_P]),
    "sporder_context_set_stream_limit": (None, [_P, C.c_uint64]),
    "sporder_context_set_ahead_threshold": (None, [_P, C.c_int64]),
    "sporder_csg_with_table": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, _P, C.c_bool, C.c_int32,
                                           C.c_float, C.c_int32, _P, _P, C.c_uint64,
                                           C.POINTER(CsgTiming), C.POINTER(CsgStats)]),
    "sporder_csg_shard": (C.c_int32, [_P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P,
                                      C.c_int32, C.c_float, C.c_int32, _P, _P, C.c_uint64,
                                      C.POINTER(CsgTiming), C.POINTER(CsgStats)]),
    "sporder_chunk_similarity_greedy_host": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, _P,
                                                         C.c_bool, C.c_int32, C.c_float, C.c_int32,
                                                         _P, C.POINTER(CsgTiming),
                                                         C.POINTER(CsgStats)]),
    "sporder_spmm": (C.c_int32, [_P, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P]),
    "sporder_spmm_async": (C.c_int32, [_P, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P]),
    "sporder_spmm_static": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, _P]),
    "sporder_kernel_launches": (C.c_uint64, []),
    "sporder_chunk_greedy": (None, [_P, C.c_int32, C.c_int32, _P, _P, C.c_bool, C.c_int32, C.c_float,
                                    C.c_int32, _P, C.POINTER(CsgTiming), C.POINTER(CgStats)]),
    "sporder_similarity_graph": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, _P, C.c_bool, C.c_int32,
                                             C.c_float, _P, _P, C.POINTER(SimTiming),
                                             C.POINTER(SimStats)]),
    "sporder_count_pillars": (None, [_P, C.c_int32, C.c_int32, _P, _P, C.c_int32,
                                     C.POINTER(C.c_int32)]),
}


def load():
    """Load the library (once) and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "chunkedgreedy_b200: %s is missing; build it with "
            "`python -m chunkedgreedy_b200.build` (there is no CPU fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # raises AttributeError when a symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error():
    msg = load().sporder_last_error()
    return msg.decode() if msg else None


def check():
    """Raise RuntimeError if the last call on this thread failed."""
    msg = last_error()
    if msg:
        raise RuntimeError("sporder_b200: " + msg)
