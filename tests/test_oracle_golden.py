"""The CPU oracle against everything that pins it (no GPU):

* the reference's only known-answer (docs/source/ex_opt_toy.rst:21);
* fixtures produced by the reference's Python CPU path (ref_py_*.npz);
* fixtures produced by the reference's CUDA extension on a B200
  (ref_cuda_*.npz).  Leaf ids and queried values must be bit-exact; colours
  agree to 1e-6 (the oracle's libm expf and CUDA's expf differ in the last
  bits, everything that decides WHERE a sample lies is bit-identical).
  Gradients agree to 1e-3 of the summed magnitude per element: the last bit
  of expf is amplified by the cancellations in ``1 - att`` and in
  ``colour * T - accum`` (rt_kernel.cu:379,467), and the fixture is one
  sample of a float-atomics sum.  (The CUDA kernels, which share CUDA's
  expf with the reference, are held to 1e-4 in the GPU tests.)
"""
import os

import numpy as np
import pytest
import torch

import parity_util as P
import svox_b200 as svox
from golden.cases import BIG, CASES
from oracle import oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")
RGB_TOL_CUDA = 1e-6     # oracle vs reference CUDA
RGB_TOL_PY = 1e-5       # oracle vs reference Python path (different clamp, fp32 reciprocal)
GRAD_REL_TOL = 1e-3    # oracle (libm) vs reference CUDA, see above


def _fixture(kind, name):
    path = os.path.join(GOLD, f"{kind}_{name}.npz")
    if not os.path.exists(path):
        pytest.skip(f"no fixture {os.path.basename(path)}")
    return np.load(path)


def _check_grad(res, z, rel_tol=GRAD_REL_TOL, slack=1.0):
    # element-wise |g - ref| <= rel_tol * sum|contributions| on the fixture's sample
    grad, idx = res["grad"], z["grad_idx"]
    worst = P.grad_excess(grad.reshape(-1)[idx], z["grad_val"], res["grad_abs"].reshape(-1)[idx],
                          rel_tol)
    assert worst <= slack, f"gradient off by {worst:.2f} x tolerance"
    assert abs(grad.sum() - float(z["grad_sum"])) <= 1e-4 * float(z["grad_abs_sum"])
    assert abs(np.abs(grad).sum() - float(z["grad_abs_sum"])) <= 1e-4 * float(z["grad_abs_sum"])


def test_known_answer_toy_example():
    # one root cell with sigma 0.5 and zero colour coefficient, ray along +z
    t = svox.N3Tree(data_format="SH1")
    with torch.no_grad():           # the leaf containing world point (0, 0, 0)
        t.data[0, 0, 0, 0, :-1] = 0.0
        t.data[0, 0, 0, 0, -1:] = 0.5
    o = np.array([[0.1, 0.1, -0.1]], np.float32)
    d = np.array([[0.0, 0.0, 1.0]], np.float32)
    out = orc.volume_render(orc.Tree.from_n3tree(t), o, d, d, orc.options(basis_dim=1))
    assert np.allclose(out, 0.88920575, atol=5e-8)
    # closed form: T = exp(-sigma * (0.5 + step)), colour 1/2, white background
    T = np.exp(-0.5 * (0.5 + 1e-3))
    assert np.allclose(out, 0.5 * (1 - T) + T, atol=1e-6)


@pytest.mark.parametrize("name", [n for n in CASES if n not in BIG])
def test_oracle_vs_reference_cuda(name):
    z = _fixture("ref_cuda", name)
    case = CASES[name]()
    res = P.run_oracle(case)
    if case["kind"] == "query":
        assert np.array_equal(res["ids"], z["ids"])
        assert np.array_equal(res["out"][:P.QUERY_ROWS_KEPT], z["out"])
        flat = case["tree"].data.detach().numpy().reshape(-1, case["tree"].data_dim)
        assert np.array_equal(res["out"], flat[res["ids"]])
    else:
        assert np.abs(res["out"] - z["out"]).max() <= RGB_TOL_CUDA
    if "grad_idx" in z.files:
        _check_grad(res, z)
        if "grad_val2" in z.files:
            # the yardstick of the GPU tests: the reference against its own second run on the
            # same inputs meets the tolerance the kernels are held to, with room to spare
            idx = z["grad_idx"]
            maxnorm, worst = P.grad_deviation(z["grad_val2"], z["grad_val"],
                                              res["grad_abs"].reshape(-1)[idx])
            assert maxnorm <= 0.1 * P.GRAD_MAXNORM_TOL and worst <= 0.1


def test_reference_does_not_reproduce_itself_elementwise():
    # Why the GPU tests do not assert a plain element-wise relative error: recorded in the
    # fixtures (spread_rel) is the largest |g1 - g2| / |g1| between two runs of the reference's
    # own CUDA backward over elements with |g1| > 1e-6 max|g1|.  For the full-size training step
    # it is far above 1e-4 (cancelling float atomics), while the whole gradient agrees to 1e-7
    # of its largest element.
    z = _fixture("ref_cuda", "c4_full_rays")
    assert float(z["spread_rel"]) > 1e-3
    assert float(z["spread_maxnorm"]) < 1e-6
    worst = max(float(_fixture("ref_cuda", n)["spread_rel"]) for n in CASES
                if n not in BIG and "spread_rel" in _fixture("ref_cuda", n).files)
    assert worst > 1e-4


@pytest.mark.parametrize("name", ["c1_rays", "shell_sh9_rays", "rgba_rays", "sh1_rays",
                                  "sh25_rays", "query_c1", "query_shell"])
def test_oracle_vs_reference_python(name):
    z = _fixture("ref_py", name)
    case = CASES[name]()
    res = P.run_oracle(case)
    if case["kind"] == "query":
        assert np.array_equal(res["ids"], z["ids"])
        assert np.array_equal(res["out"][:P.QUERY_ROWS_KEPT], z["out"])
        _check_grad(res, z, rel_tol=1e-5)
    else:
        # The Python path takes one sample even when a ray misses the cube;
        # compare the rays that enter it.
        hit = P.run_oracle(case, backward=False, want_counts=True)["visits"] > 0
        err = np.abs(res["out"] - z["out"])[hit]
        assert err.max() <= (1e-4 if name == "shell_sh9_rays" else RGB_TOL_PY)
        assert np.median(err) <= 1e-6
        if hit.all():
            _check_grad(res, z, rel_tol=2e-3)


def test_big_case_config4_sample():
    """First 2^14 rays of the benchmark's training batch on the full tree."""
    z = _fixture("ref_cuda", "c4_sample_rays")
    case = CASES["c4_sample_rays"]()
    res = P.run_oracle(case, backward=False, want_counts=True)
    assert np.abs(res["out"] - z["out"]).max() <= RGB_TOL_CUDA
    # workload statistics quoted in the design notes
    assert 150 < res["visits"].mean() < 175 and 60 < res["contrib"].mean() < 75


def test_trace_log_consistency():
    case = CASES["shell_sh9_rays"]()
    ot = orc.Tree.from_n3tree(case["tree"])
    opt = orc.options(basis_dim=9)
    o, d, v = [t.numpy() for t in case["rays"]]
    out, vis, _ = orc.volume_render(ot, o, d, v, opt, want_counts=True)
    for i in (0, 17, 4000):
        slots, dts, ts, rgb = orc.trace_log(ot, o[i], d[i], v[i], opt)
        assert len(slots) == vis[i]
        assert np.array_equal(rgb, out[i])
        assert (dts > 0).all() and (np.diff(ts) > 0).all()
        assert (case["tree"].child.reshape(-1)[torch.from_numpy(slots)] == 0).all()


def test_corrupt_tree_is_reported_not_followed():
    t = svox.N3Tree(init_refine=1, data_format="SH1")
    child = t.child.numpy().copy()
    child[0, 0, 0, 0] = 10_000           # link far outside the node array
    ot = orc.Tree(t.data.detach().numpy(), child)
    with pytest.raises(RuntimeError, match="corrupt"):
        orc.query_vertical(ot, np.array([[0.1, 0.1, 0.1]], np.float32))


def test_weight_accumulation_matches_a_per_ray_recomputation():
    # svox/csrc/rt_kernel.cu:298-304: every contributing sample adds light * (1 - att) to its
    # leaf.  Recompute that from the oracle's own per-visit log for a few rays of config 1
    # (unit cube, unit directions: delta_scale = 1).
    from oracle import oracle as orc
    case = CASES["c1_rays"]()
    tree = orc.Tree.from_n3tree(case["tree"])
    opt = orc.options(basis_dim=4)
    o, d, v = [t.numpy()[:8] for t in case["rays"]]
    with orc.weight_accumulation(tree, "sum") as acc_sum:
        orc.volume_render(tree, o, d, v, opt)
    with orc.weight_accumulation(tree, "max") as acc_max:
        orc.volume_render(tree, o, d, v, opt)
    want_sum = np.zeros(acc_sum.size)
    want_max = np.zeros(acc_sum.size)
    sigma = tree.data.reshape(-1, tree.K)[:, -1]
    for i in range(8):
        slots, dts, _, _ = orc.trace_log(tree, o[i], d[i], v[i], opt)
        light = np.float32(1.0)
        for s_, dt in zip(slots, dts):
            sg = sigma[s_]
            if sg > 0:
                att = np.exp(np.float32(-dt) * np.float32(1.0) * sg, dtype=np.float32)
                w = light * (np.float32(1.0) - att)
                want_sum[s_] += float(w)
                want_max[s_] = max(want_max[s_], float(w))
                light = light * att
    assert want_sum.sum() > 1.0
    assert np.abs(acc_sum.reshape(-1) - want_sum).max() < 1e-6
    assert np.abs(acc_max.reshape(-1) - want_max).max() < 1e-6


@pytest.mark.parametrize("name", ["c1_rays", "shell_sh9_rays", "shell_sh16_image", "rgba_rays"])
def test_weight_accumulation_against_reference_cuda_fixture(name):
    # Fixtures: the reference's CUDA extension with tree._weight_accum switched on
    # (tests/golden/make_ref_cuda_golden.py --weights).
    z = np.load(os.path.join(GOLD, f"ref_cuda_weights_{name}.npz"))
    case = CASES[name]()
    for op in ("sum", "max"):
        mine = P.run_weight_accumulation(case, op)
        assert mine.size == int(z["size"])
        want = np.zeros(mine.size)
        want[z["idx"]] = z[op]
        tol = 1e-5 * (1.0 + np.abs(want)) if op == "sum" else 2e-6
        assert np.all(np.abs(mine - want) <= tol), np.abs(mine - want).max()


@pytest.mark.parametrize("name", ["c1_rays", "opt_comp_range", "shell_sh16_image", "sg9_rays",
                                  "asg4_rays", "rgba_rays", "n3_rays"])
def test_se_grad_against_reference_cuda_fixture(name):
    # Fixtures: the reference's se_grad / se_grad_persp (CUDA) on seeded colours
    # (tests/golden/make_ref_cuda_golden.py --se-grad).
    z = np.load(os.path.join(GOLD, f"ref_cuda_se_grad_{name}.npz"))
    case = CASES[name]()
    mine = P.run_se_grad(case, "oracle")
    assert np.abs(mine["out"] - z["out"]).max() <= 1e-5
    gi, hi = z["grad_idx"], z["hess_idx"]
    worst = P.grad_excess(mine["grad"].reshape(-1)[gi], z["grad_val"],
                          mine["grad_abs"].reshape(-1)[gi], 1e-3)
    assert worst <= 1.0, worst
    h, want = mine["hess"].reshape(-1)[hi], z["hess_val"]
    # (with density_softplus the reference's diagonal has a signed term: entries can be negative)
    assert np.all(np.abs(h - want) <= 1e-3 * np.abs(want) + 1e-4 * np.abs(want).max())
    assert abs(mine["hess"].sum() - float(z["hess_sum"])) <= 1e-3 * float(z["hess_abs_sum"])
