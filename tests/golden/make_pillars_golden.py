"""Records the reference library's pillar counts (sporder_count_pillars of the unmodified
reference sources built by oracle/build_ref.sh) for the cases of tests/cases.py.

Needs a GPU and oracle/_ref/libsporder_ref.so.  usage:
    python tests/golden/make_pillars_golden.py [output.json]
The committed tests/golden/pillars_golden.json was written by this script on a B200.
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import torch  # noqa: E402

import cases  # noqa: E402
from oracle import ref  # noqa: E402

HEIGHTS = (1, 2, 7, 16, 32, 100, 1024)


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "pillars_golden.json")
    out = {}
    for name in cases.CASES:
        ptr, ind, val, sym, params = cases.build(name)
        d_ptr, d_ind = torch.from_numpy(ptr).cuda(), torch.from_numpy(ind).cuda()
        out[name] = {str(h): ref.count_pillars(d_ptr, d_ind, h) for h in HEIGHTS}
    with open(out_path, "w") as f:
        json.dump(out, f, indent=0, sort_keys=True)
    print("wrote", out_path, len(out), "cases")


if __name__ == "__main__":
    main()
