"""Host logic: tree construction, refinement order, views, persistence (no GPU)."""
import numpy as np
import pytest
import torch

import svox_b200 as svox
from svox_b200 import workloads as W


def test_uniform_counts_and_depth_numbering():
    # "refined to depth d" with (2^d)^3 leaves == init_refine = d - 1
    t = svox.N3Tree(init_refine=3, data_format="SH4")
    assert (t.n_internal, t.n_leaves, t.capacity) == (585, 4096, 585)
    assert t.max_depth == 3
    assert t.data.shape == (585, 2, 2, 2, 13) and t.child.dtype == torch.int32
    t.check_integrity()


def test_refine_numbering_contract():
    # new nodes are appended in selector order; children are relative offsets
    t = svox.N3Tree(init_refine=0)
    assert t.n_internal == 1 and (t.child == 0).all()
    t.refine()
    assert t.n_internal == 9
    assert t.child[0].reshape(-1).tolist() == list(range(1, 9))
    assert t.parent_depth[1:9, 0].tolist() == list(range(8))
    # stored depth: root 0, its child nodes 1 (a leaf reports the depth of its node)
    assert t.parent_depth[1:9, 1].tolist() == [1] * 8
    # refine only the leaf (node 3, cell (1,0,1)): new node 9, link is relative
    sel = (torch.tensor([3]), torch.tensor([1]), torch.tensor([0]), torch.tensor([1]))
    t.refine(sel=sel)
    assert t.n_internal == 10 and t.child[3, 1, 0, 1].item() == 9 - 3
    assert t.parent_depth[9].tolist() == [3 * 8 + 5, 2]
    t.check_integrity()


def test_refine_repeats_equals_sequential():
    a = svox.N3Tree(init_refine=1)
    b = svox.N3Tree(init_refine=1)
    m = torch.zeros(a.n_leaves, dtype=torch.bool)
    m[[3, 17, 40]] = True
    a[m].refine(2)
    b[m].refine(1)
    # second level: the cells of the three new nodes, in order
    new = torch.arange(b.n_internal - 3, b.n_internal)
    leaves = b._all_leaves()
    pick = torch.isin(leaves[:, 0], new)
    b[pick].refine(1)
    assert torch.equal(a.child, b.child) and torch.equal(a.parent_depth, b.parent_depth)


def test_refine_respects_depth_limit_and_inherits_values():
    t = svox.N3Tree(init_refine=0, depth_limit=1, data_format="SH1")
    with torch.no_grad():
        t.data[0] = torch.arange(8.0).reshape(2, 2, 2, 1).expand(2, 2, 2, 4)
    t.refine()
    assert t.n_internal == 9
    assert (t.data[1 + 5] == 5.0).all()       # children copy the parent's record
    # the new nodes sit at the depth limit: nothing left to refine
    assert t.refine() is False and t.n_internal == 9
    assert t.max_depth == 1


def test_pack_unpack_roundtrip():
    t = svox.N3Tree(N=3, init_refine=1)
    ids = torch.arange(0, t.n_internal * 27, 7)
    assert torch.equal(t._pack_index(t._unpack_index(ids.clone())), ids)


def test_view_geometry():
    t = svox.N3Tree(init_refine=1, radius=[1.0, 2.0, 4.0], center=[1.0, 0.0, -1.0])
    v = t[:]
    assert v.depths.tolist() == [1] * 64
    assert torch.allclose(v.lengths_local, torch.full((64,), 0.25))
    assert torch.allclose(v.lengths, torch.tensor([0.5, 1.0, 2.0]).expand(64, 3))
    c = v.corners_local
    assert c.min() == 0 and c.max() == 0.75 and torch.unique(c, dim=0).shape[0] == 64
    w = v.corners
    assert torch.allclose(w.min(0).values, torch.tensor([0.0, -2.0, -5.0]))
    p = torch.rand(5, 3)
    assert torch.allclose(t.world2tree(t.tree2world(p)), p, atol=1e-6)


def test_view_set_get_and_channel_key():
    t = svox.N3Tree(init_refine=1, data_format="SH1")
    t[:] = 2.0
    assert (t[:].values == 2.0).all()
    t[:, -1:] = 7.0
    assert (t.data[1:, ..., -1] == 7.0).all() and (t.data[1:, ..., 0] == 2.0).all()
    m = torch.zeros(64, dtype=torch.bool)
    m[5] = True
    t[m] = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    assert t[5].values.tolist() == [1.0, 2.0, 3.0, 4.0]
    assert (t[:] + 1).shape == (64, 4)
    v = t[:]
    t.refine()
    with pytest.raises(RuntimeError, match="invalidated"):
        v.values


def test_save_load_roundtrip(tmp_path):
    gen = torch.Generator().manual_seed(5)
    t = W.uniform_tree(2, "SH4", gen, sigma_range=(0, 5))
    p = str(tmp_path / "tree.npz")
    t.save(p)
    z = np.load(p)
    assert set(z.files) >= {"data_dim", "child", "parent_depth", "n_internal", "n_free",
                            "invradius3", "offset", "depth_limit", "geom_resize_fact", "data",
                            "data_format"}
    assert z["data"].dtype == np.float16          # the file format stores half precision
    u = svox.N3Tree.load(p)
    assert torch.equal(u.child, t.child) and torch.equal(u.parent_depth, t.parent_depth)
    assert torch.allclose(u.data, t.data, atol=2e-2, rtol=1e-3)
    assert repr(u.data_format) == "SH4" and u.n_internal == t.n_internal


def test_config4_structure_small():
    # same construction as the benchmark tree, two levels shallower
    tree, rays, targets = W.config4(Q=64, init_refine=3, extra_levels=3)
    tree.check_integrity()
    d = tree[:].depths
    assert d.min() == 3 and d.max() == 6
    sig = tree[:].values[:, -1]
    assert (sig[d < 6] == 0).all() and (sig > 0).any() and sig.max() <= 50
    assert torch.allclose(rays.dirs.norm(dim=1), torch.ones(64), atol=1e-6)
    assert targets.shape == (64, 3)


def test_state_dict_names():
    t = svox.N3Tree(init_refine=1)
    assert set(t.state_dict()) == {"data", "child", "parent_depth", "_n_internal", "_n_free",
                                   "invradius", "offset"}
