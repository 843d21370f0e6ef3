"""Generate fixtures from the reference's own Python (CPU tensor) path.

Imports the unmodified reference package from a checkout (first argument, or
the default below; it has no compiled extension there, so every call takes the
pure-PyTorch path of svox/svox.py:224-268 and svox/renderer.py:205-282) and
stores its outputs for the seeded cases it can express: zero thresholds,
unit-cube world box, SH / RGBA colour.  Trees are built with the reference's
own N3Tree from the same seeds and checked to be structurally identical to
the ones tests/golden/cases.py builds.

    ref_py_<case>.npz: out, [ids], [grad_* digest]

Work-arounds that leave the reference untouched: inputs are cloned (the CPU
path normalises ``dirs`` and clamps points in place), and the background is
passed as an object whose ``__rmul__`` broadcasts per ray (the CPU path adds
a (B,) vector to a (B,3) tensor, svox/renderer.py:281).

Usage: python tests/golden/make_ref_py_golden.py [reference_root] [case ...]
"""
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.dont_write_bytecode = True

from golden.cases import CASES  # noqa: E402
import parity_util as P  # noqa: E402

PY_CASES = ["c1_rays", "shell_sh9_rays", "rgba_rays", "sh1_rays", "sh25_rays",
            "query_c1", "query_shell"]


class _Background:
    def __init__(self, v):
        self.v = v

    def __rmul__(self, t):
        return t[:, None] * self.v


def main():
    root = sys.argv[1] if len(sys.argv) > 1 and os.path.isdir(sys.argv[1]) else "/root/reference"
    names = [a for a in sys.argv[1:] if a in CASES] or PY_CASES
    sys.path.insert(0, root)
    warnings.filterwarnings("ignore")
    import svox as ref

    for name in names:
        case = CASES[name]()
        mine = case["tree"]
        # the reference's tree class, filled with the same tensors
        fmt = repr(mine.data_format)
        tree = ref.N3Tree(N=mine.N, data_format=fmt, data_dim=mine.data_dim)
        tree.data = torch.nn.Parameter(mine.data.data.clone())
        tree.child = mine.child.clone()
        tree.parent_depth = mine.parent_depth.clone()
        tree._n_internal.fill_(mine.n_internal)
        tree.invradius = mine.invradius.clone()
        tree.offset = mine.offset.clone()
        tree._invalidate()
        tree.check_integrity()
        blob = {}
        if case["kind"] == "query":
            vals, ids = tree.forward(case["points"].clone(), cuda=False, want_node_ids=True)
            blob["out"], blob["ids"] = vals.detach().numpy()[:P.QUERY_ROWS_KEPT], ids.numpy()
            vals.backward(case["grad_out"])
        else:
            po = P.options_of(case)
            assert po.sigma_thresh == 0 and po.stop_thresh == 0
            r = ref.VolumeRenderer(tree, step_size=po.step_size,
                                   background_brightness=_Background(po.background_brightness))
            rays = ref.Rays(*[t.clone() for t in case["rays"]])
            out = r(rays, cuda=False)
            blob["out"] = out.detach().numpy()
            out.backward(case["grad_out"])
        blob.update(P.grad_digest(tree.data.grad.numpy()))
        np.savez_compressed(os.path.join(HERE, f"ref_py_{name}.npz"), **blob)
        print(name, blob["out"].shape, flush=True)


if __name__ == "__main__":
    main()
