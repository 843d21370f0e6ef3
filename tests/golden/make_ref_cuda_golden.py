"""Generate the reference-CUDA fixtures (run on a machine with a GPU).

Runs the UNMODIFIED reference extension (built by oracle/build_ref.py into
oracle/_ref) on every seeded case of tests/golden/cases.py and stores its
outputs as ``ref_cuda_<case>.npz``:

    out            rendered colours (float32); for query cases the values of the
                   first QUERY_ROWS_KEPT points (the rest follow from ids)
    ids            packed leaf ids (query cases)
    grad_*         digest of the gradient w.r.t. tree.data (see
                   tests/parity_util.grad_digest)
    grad_val2      the same sampled elements from a SECOND run of the reference on the
                   same inputs: its gradient is a sum of float atomics in whatever order
                   the hardware took them, so two runs differ; the difference is the
                   yardstick for "equal up to the order of the atomics"
    spread_*       that run-to-run difference over the WHOLE gradient: largest
                   |g1 - g2| / max|g1|, and largest |g1 - g2| / |g1| over elements
                   with |g1| > 1e-6 max|g1|

and, for WEIGHT_CASES, the reference's weight accumulator after one forward
render as ``ref_cuda_weights_<case>.npz`` (non-zero entries only):

    idx            flat indices into (M, N, N, N)
    sum, max       accumulated weight per index with op "sum" / "max"

and, for SE_GRAD_CASES, the reference's se_grad / se_grad_persp on the seeded
colours of tests/parity_util.se_grad_colors as ``ref_cuda_se_grad_<case>.npz``:

    out            returned colours
    grad_*         digest of the gradient
    hess_*         digest of the Gauss-Newton diagonal

The full-size cases (FULL_CASES, "--full") keep a strided sample of the outputs
(see tests/golden/cases.py).

Usage: python tests/golden/make_ref_cuda_golden.py [out_dir] [case ...]
       python tests/golden/make_ref_cuda_golden.py [out_dir] --full
       python tests/golden/make_ref_cuda_golden.py [out_dir] --weights
       python tests/golden/make_ref_cuda_golden.py [out_dir] --se-grad [case ...]
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from golden.cases import (CASES, FULL_CASES, FULL_ID_STRIDE, FULL_OUT_STRIDE,  # noqa: E402
                          FULL_PIXEL_STRIDE)
import parity_util as P  # noqa: E402


WEIGHT_CASES = ["c1_rays", "shell_sh9_rays", "shell_sh16_image", "rgba_rays"]


def weights(out_dir):
    for name in WEIGHT_CASES:
        case = CASES[name]()
        s = P.run_ref_cuda(case, weight_op="sum")["weights"]
        m = P.run_ref_cuda(case, weight_op="max")["weights"]
        idx = np.flatnonzero((s != 0) | (m != 0)).astype(np.int64)
        np.savez_compressed(os.path.join(out_dir, f"ref_cuda_weights_{name}.npz"), idx=idx,
                            sum=s[idx].astype(np.float32), max=m[idx].astype(np.float32),
                            size=np.int64(s.size))
        print(name, "weights: non-zero", idx.size, "of", s.size, flush=True)


SE_GRAD_CASES = ["c1_rays", "shell_sh9_rays", "shell_sh16_image", "opt_comp_range",
                 "opt_softplus_pad_bg", "sg9_rays", "asg4_rays", "rgba_rays", "n3_rays",
                 "sg5_rays", "asg7_image"]


def se_grad(out_dir, names):
    for name in names or SE_GRAD_CASES:
        case = CASES[name]()
        res = P.run_se_grad(case, "ref_cuda")
        blob = {"out": res["out"]}
        blob.update(P.grad_digest(res["grad"]))
        blob.update({"hess" + k[4:]: v for k, v in P.grad_digest(res["hess"]).items()})
        np.savez_compressed(os.path.join(out_dir, f"ref_cuda_se_grad_{name}.npz"), **blob)
        print(name, "se_grad out", res["out"].shape, "grad nnz", int(blob["grad_nnz"]),
              "hess nnz", int(blob["hess_nnz"]), flush=True)


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else HERE
    os.makedirs(out_dir, exist_ok=True)
    if "--weights" in sys.argv:
        return weights(out_dir)
    if "--se-grad" in sys.argv:
        return se_grad(out_dir, [a for a in sys.argv[2:] if not a.startswith("--")])
    full = "--full" in sys.argv
    table = FULL_CASES if full else CASES
    names = [a for a in sys.argv[2:] if not a.startswith("--")] or list(table)
    for name in names:
        case = table[name]()
        res = P.run_ref_cuda(case)
        blob = {"out": res["out"]}
        if full and case["kind"] == "rays":
            blob["out"] = res["out"][::FULL_OUT_STRIDE]
        elif full and case["kind"] == "image":
            blob["out"] = res["out"].reshape(-1, res["out"].shape[-1])[::FULL_PIXEL_STRIDE]
        if res["ids"] is not None:
            blob["ids"] = res["ids"][::FULL_ID_STRIDE] if full else res["ids"]
            blob["out"] = res["out"][:P.QUERY_ROWS_KEPT]
        if res["grad"] is not None:
            blob.update(P.grad_digest(res["grad"]))
            g1 = res["grad"].reshape(-1)
            g2 = P.run_ref_cuda(case)["grad"].reshape(-1)       # the same again
            blob["grad_val2"] = g2[blob["grad_idx"]]
            diff, top = np.abs(g1 - g2), np.abs(g1).max()
            big = np.abs(g1) > 1e-6 * top
            blob["spread_maxnorm"] = diff.max() / top
            blob["spread_rel"] = (diff[big] / np.abs(g1[big])).max() if big.any() else 0.0
            print(name, "run-to-run: max-norm %.3g, element-wise %.3g" %
                  (blob["spread_maxnorm"], blob["spread_rel"]), flush=True)
        np.savez_compressed(os.path.join(out_dir, f"ref_cuda_{name}.npz"), **blob)
        print(name, "out", res["out"].shape, "grad", None if res["grad"] is None
              else res["grad"].shape, flush=True)


if __name__ == "__main__":
    main()
