"""Records outputs of the REFERENCE library for the cases of tests/cases.py.

Run on a machine with a GPU and the reference build (oracle/_ref/libsporder_ref.so,
made by oracle/build_ref.sh from the unmodified reference sources):

    python tests/golden/make_golden.py [out_dir]

Writes csg_golden.npz: per case the permutation of sporder_chunk_similarity_greedy,
the internal top-k table (through oracle/ref_shim.cu), and the symmetric reorder of the
matrix by that permutation (ptr, ind, val) from sporder_reorder.  The committed copy
of that file is what pins the CPU oracle (tests/test_oracle_golden.py).
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

import torch  # noqa: E402

import cases  # noqa: E402
import oracle  # noqa: E402
from oracle import ref  # noqa: E402


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(out_dir, exist_ok=True)
    out = {}
    for name in cases.CASES:
        ptr, ind, val, sym, params = cases.build(name)
        n, nnz = ptr.size - 1, ind.size
        prm = oracle.resolve_params(n, nnz, **params)
        dp = torch.from_numpy(ptr).cuda()
        di = torch.from_numpy(ind).cuda()
        dv = torch.from_numpy(val).cuda()
        order = ref.csg(dp, di, sym, **params)
        table = ref.csg_table(dp, di, sym, prm["k"], prm["oversampling"], prm["chunk_size"])
        rp, ri, rv = ref.reorder(dp, di, order, dv, symmetric=True)
        torch.cuda.synchronize()
        out[name + "/order"] = order.cpu().numpy()
        tab = table.cpu().numpy().view(np.uint64)
        out[name + "/table_sha256"] = np.frombuffer(
            hashlib.sha256(np.ascontiguousarray(tab).tobytes()).digest(), dtype=np.uint8)
        if n <= 2048:
            out[name + "/table"] = tab
        out[name + "/sym_ptr"] = rp.cpu().numpy()
        out[name + "/sym_ind_sha256"] = np.frombuffer(
            hashlib.sha256(ri.cpu().numpy().tobytes()).digest(), dtype=np.uint8)
        out[name + "/sym_val_sha256"] = np.frombuffer(
            hashlib.sha256(rv.cpu().numpy().tobytes()).digest(), dtype=np.uint8)
        out[name + "/shape"] = np.array([n, nnz, prm["k"], prm["M"], prm["chunk_size"]],
                                        dtype=np.int64)
        print(name, n, nnz, prm)
    path = os.path.join(out_dir, "csg_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
