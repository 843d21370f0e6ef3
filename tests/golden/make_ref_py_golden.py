"""Generate fixtures from the reference's own Python (CPU tensor) path.

Imports the unmodified reference package from a checkout (first argument, or
the default below; it has no compiled extension there, so every call takes the
pure-PyTorch path of svox/svox.py:224-268 and svox/renderer.py:205-282) and
stores its outputs for the seeded cases it can express: zero thresholds,
unit-cube world box, SH / RGBA colour.  For these the tensors of the trees
that tests/golden/cases.py builds are copied into the reference's N3Tree class
(so both sides render the same bits).

    ref_py_<case>.npz: out, [ids], [grad_* digest]

With ``--structure`` it instead builds trees with the REFERENCE's own
constructor, ``refine`` and view selection, and writes them with the
reference's own ``N3Tree.save``:

    ref_py_saved_tree_<name>.npz   (the reference's checkpoint format, as written by it)

and, next to each, ``ref_py_frontier_<name>.npz``: the reference's frontier queries, the
corners and side lengths of every leaf (its tensor-op ``_calc_corners``), a point assignment
``tree.set(points, values, cuda=False)`` (the rows of ``data`` it changed), the first records of
``tree.clone().expand(...)`` and ``tree.partial(-1)``, and the selection of a merge whose result
is ``ref_py_saved_tree_<name>_merged.npz``.

tests/test_tree_structure.py loads those files with svox_b200.N3Tree.load,
rebuilds the same trees with svox_b200 from the same recipe (RECIPES below)
and compares node numbering and file contents.

Work-arounds that leave the reference untouched: inputs are cloned (the CPU
path normalises ``dirs`` and clamps points in place), and the background is
passed as an object whose ``__rmul__`` broadcasts per ray (the CPU path adds
a (B,) vector to a (B,3) tensor, svox/renderer.py:281).

Usage: python tests/golden/make_ref_py_golden.py [reference_root] [case ...]
       python tests/golden/make_ref_py_golden.py [reference_root] --structure
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


# Recipes of the structure fixtures.  Either library follows them with its own N3Tree:
# constructor, then for every (lo, hi, repeats): refine `repeats` times the leaves whose
# centre lies at distance [lo, hi] from the centre of the cube, then seeded values.
RECIPES = {
    "octree": dict(ctor=dict(N=2, data_format="SH4", init_refine=2),
                   refines=[(0.25, 0.40, 2), (0.30, 0.33, 1)], seed=201),
    "n3": dict(ctor=dict(N=3, data_format="RGBA", init_refine=1, radius=[0.5, 1.0, 2.0],
                         center=[0.0, 0.5, -1.0]),
               refines=[(0.0, 0.30, 1)], seed=202),
}


# the layout each recipe tree is expanded to for the `expand_*` entries of the frontier fixture
EXPANDED = {"octree": "SH9", "n3": "SH1"}


def build_recipe(lib, recipe):
    """``lib``: the reference package or svox_b200 (same API)."""
    tree = lib.N3Tree(**recipe["ctor"])
    for lo, hi, repeats in recipe["refines"]:
        view = tree[:]
        centre = view.corners_local + 0.5 * view.lengths_local[:, None]
        dist = (centre - 0.5).norm(dim=1)
        tree[(dist >= lo) & (dist <= hi)].refine(repeats)
    gen = torch.Generator().manual_seed(recipe["seed"])
    with torch.no_grad():
        tree.data.data.copy_(torch.randn(tree.data.shape, generator=gen))
    return tree


def assignment(recipe, n_leaves):
    """Seeded inputs of the ``tree.set`` fixture: one point inside every third leaf is not
    expressible without the tree, so points are uniform in the world box, few enough that
    hardly any two share a leaf; the caller drops those that do."""
    gen = torch.Generator().manual_seed(recipe["seed"] + 1000)
    ctor = recipe["ctor"]
    radius = torch.as_tensor(ctor.get("radius", 0.5), dtype=torch.float32).expand(3)
    center = torch.as_tensor(ctor.get("center", [0.5, 0.5, 0.5]), dtype=torch.float32)
    Q = max(8, n_leaves // 6)
    pts = center + (torch.rand(Q, 3, generator=gen) * 2 - 1) * radius * 0.999
    return pts, gen


def coarsen(tree):
    """The merge both libraries perform on a recipe tree: every second frontier node whose
    largest last-channel value is below the median goes back into its parent (mean of the
    children), then the arrays are compacted."""
    top = tree.max_frontier(dim=-1)
    pick = torch.zeros(tree.n_frontier, dtype=torch.bool)
    pick[::2] = True
    pick &= top <= top.median()
    tree.merge(pick)
    tree.shrink_to_fit()
    return pick


def structure(ref):
    for name, recipe in RECIPES.items():
        tree = build_recipe(ref, recipe)
        tree.check_integrity()
        path = os.path.join(HERE, f"ref_py_saved_tree_{name}.npz")
        tree.save(path)                      # the reference's own writer
        print(name, "nodes", tree.n_internal, "leaves", tree.n_leaves, "->", path, flush=True)
        # frontier queries and a merge + compaction, all by the reference's own code
        blob = dict(frontier=tree._frontier.numpy(), frontier_depth=tree.frontier_depth.numpy(),
                    mean=tree.reduce_frontier().numpy(), top=tree.max_frontier(dim=-1).numpy(),
                    diam=tree.diam_frontier().numpy())
        # geometry of every leaf, and a point assignment (tree.set), by the reference's CPU path
        view = tree[:]
        blob["leaf_corners"] = view.corners_local.numpy()
        blob["leaf_lengths"] = view.lengths_local.numpy()
        pts, gen = assignment(recipe, tree.n_leaves)
        _, ids = tree.forward(pts.clone(), cuda=False, want_node_ids=True)
        _, first = np.unique(ids.numpy(), return_index=True)      # one point per leaf
        pts = pts[np.sort(first)]
        vals = torch.randn(pts.shape[0], tree.data_dim, generator=gen)
        before = tree.data.data.clone()
        tree.set(pts.clone(), vals, cuda=False)
        blob["set_points"], blob["set_values"] = pts.numpy(), vals.numpy()
        after = tree.data.data.reshape(-1, tree.data_dim)
        rows = (after != before.reshape(-1, tree.data_dim)).any(dim=1).nonzero()[:, 0]
        blob["set_rows"], blob["set_rows_data"] = rows.numpy(), after[rows].numpy().copy()
        tree.data.data.copy_(before)
        # a copy with another record layout (clone + expand), and the densities alone (partial)
        wider = tree.clone()
        wider.expand(EXPANDED[name])
        blob["expand_rows"] = wider.data.data.reshape(-1, wider.data_dim)[:64].numpy().copy()
        blob["expand_sum"] = wider.data.data.double().sum().numpy()
        blob["partial_rows"] = tree.partial(-1, data_format="RGBA").data.data.reshape(-1)[:64] \
            .numpy().copy()
        blob["pick"] = coarsen(tree).numpy()
        tree.check_integrity()
        np.savez_compressed(os.path.join(HERE, f"ref_py_frontier_{name}.npz"), **blob)
        tree.save(os.path.join(HERE, f"ref_py_saved_tree_{name}_merged.npz"), shrink=False)
        print(name, "merged", int(blob["pick"].sum()), "of", blob["pick"].size,
              "frontier nodes ->", tree.n_internal, "nodes", flush=True)


def main():
    from oracle.build_ref import reference_root
    root = sys.argv[1] if len(sys.argv) > 1 and os.path.isdir(sys.argv[1]) else reference_root()
    names = [a for a in sys.argv[1:] if a in CASES] or PY_CASES
    sys.path.insert(0, root)
    warnings.filterwarnings("ignore")
    import svox as ref
    if "--structure" in sys.argv:
        return structure(ref)

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
