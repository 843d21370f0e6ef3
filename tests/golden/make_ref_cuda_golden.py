"""Generate the reference-CUDA fixtures (run on a machine with a GPU).

Runs the UNMODIFIED reference extension (built by oracle/build_ref.py into
oracle/_ref) on every seeded case of tests/golden/cases.py and stores its
outputs as ``ref_cuda_<case>.npz``:

    out            rendered colours (float32); for query cases the values of the
                   first QUERY_ROWS_KEPT points (the rest follow from ids)
    ids            packed leaf ids (query cases)
    grad_*         digest of the gradient w.r.t. tree.data (see
                   tests/parity_util.grad_digest)

Usage: python tests/golden/make_ref_cuda_golden.py [out_dir] [case ...]
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from golden.cases import CASES  # noqa: E402
import parity_util as P  # noqa: E402


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    names = sys.argv[2:] or list(CASES)
    os.makedirs(out_dir, exist_ok=True)
    for name in names:
        case = CASES[name]()
        res = P.run_ref_cuda(case)
        blob = {"out": res["out"]}
        if res["ids"] is not None:
            blob["ids"] = res["ids"]
            blob["out"] = res["out"][:P.QUERY_ROWS_KEPT]
        if res["grad"] is not None:
            blob.update(P.grad_digest(res["grad"]))
        np.savez_compressed(os.path.join(out_dir, f"ref_cuda_{name}.npz"), **blob)
        print(name, "out", res["out"].shape, "grad", None if res["grad"] is None
              else res["grad"].shape, flush=True)


if __name__ == "__main__":
    main()
