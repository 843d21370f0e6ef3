"""Parity at the benchmark configurations' full sizes -- needs a GPU (and about 40 GB of host
memory for the largest tree and the oracle's double-precision gradients).

Each test runs the CUDA path on the whole workload and compares it with
* the fixture of the reference's CUDA extension for the same seeded inputs
  (tests/golden/ref_cuda_*_full_*.npz: a strided sample of the outputs, a sample of the
  gradient from two runs of the reference), and
* the CPU oracle on a sample the oracle finishes in seconds, or a closed form.

What the full sizes exercise that the small cases cannot: byte offsets into ``data`` beyond
2^31 (query, 3.76 GB) and element offsets beyond 2^31 (the 12 GB tree), millions of log
chunks and every bin of the replay backward at full occupancy.
"""
import os

import numpy as np
import pytest
import torch

import parity_util as P
import svox_b200 as svox
from golden.cases import (FULL_CASES, FULL_ID_STRIDE, FULL_OUT_STRIDE, FULL_PIXEL_STRIDE)
from svox_b200 import csrc

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
RGB_TOL = 1e-5


def _gold(name):
    path = os.path.join(GOLD, f"ref_cuda_{name}.npz")
    return np.load(path) if os.path.exists(path) else None


def test_training_step_full_size(cuda_device):
    # 2^20 rays on the 512^3 shell tree, MSE against the seeded targets: the logged forward
    # and the replay backward at the size the benchmark times them.
    case = FULL_CASES["c4_full_rays"]()
    z = _gold("c4_full_rays")
    assert z is not None
    mine = P.run_product(case, cuda_device)
    assert np.abs(mine["out"][::FULL_OUT_STRIDE] - z["out"]).max() <= RGB_TOL
    orc = P.run_oracle(case)                      # for the per-element scale of the tolerance
    assert np.abs(mine["out"] - orc["out"]).max() <= RGB_TOL
    idx = z["grad_idx"]
    g = mine["grad"].reshape(-1)[idx]
    scale = orc["grad_abs"].reshape(-1)[idx]
    maxnorm, worst = P.assert_grad_matches_reference(g, z["grad_val"], scale, "training step")
    # the reference against its own second run, same yardstick
    ref_maxnorm, ref_worst = P.grad_deviation(z["grad_val2"], z["grad_val"], scale)
    print(f"full-size gradient: max-norm {maxnorm:.2e} (reference vs itself {ref_maxnorm:.2e}), "
          f"worst element {worst:.3f} of its allowance (reference vs itself {ref_worst:.3f})")
    assert P.grad_excess(mine["grad"], orc["grad"], orc["grad_abs"], 1e-3) <= 1.0
    total = float(z["grad_abs_sum"])
    assert abs(np.abs(mine["grad"]).sum() - total) <= 1e-5 * total
    # the marching backward (no item log) gives the same gradient at this size too
    march = P.run_product(case, cuda_device, item_log=False)
    P.assert_grad_matches_reference(march["grad"].reshape(-1)[idx], z["grad_val"], scale,
                                    "marching backward")


def test_query_full_size(cuda_device):
    # 2^24 points on 256^3 leaves with 49 floats each: 3.76 GB of data (byte offsets > 2^31),
    # 3.3 GB of values.
    case = FULL_CASES["c2_full_query"]()
    z = _gold("c2_full_query")
    tree = case["tree"].to(cuda_device)
    try:
        pts = case["points"].to(cuda_device)
        tree.zero_grad(set_to_none=True)
        vals, ids = tree(pts, want_node_ids=True)
        flat = tree.data.view(-1, tree.data_dim)
        assert torch.equal(flat[ids], vals)                       # values == data[ids]
        # uniform tree: the leaf of a point is known in closed form
        cell = (pts * 256).long().clamp_(max=255)
        leaves = tree[:]
        corner = (leaves.corners_local * 256).round().long().to(cuda_device)
        lut = torch.empty(256, 256, 256, dtype=torch.int64, device=cuda_device)
        lut[corner[:, 0], corner[:, 1], corner[:, 2]] = tree._pack_index(
            tree._all_leaves().to(cuda_device))
        assert torch.equal(lut[cell[:, 0], cell[:, 1], cell[:, 2]], ids)
        assert (ids.max().item() + 1) * tree.data_dim * 4 > 2 ** 31   # the offsets are that large
        del lut, corner, cell
        if z is not None:                                         # the reference's CUDA extension
            assert np.array_equal(ids[::FULL_ID_STRIDE].cpu().numpy(), z["ids"])
            assert np.array_equal(vals[:P.QUERY_ROWS_KEPT].detach().cpu().numpy(), z["out"])
        gout = case["grad_out"].to(cuda_device)
        vals.backward(gout)
        grad = tree.data.grad.view(-1, tree.data_dim)
        # every leaf's gradient row is the sum of the upstream rows of its points
        want = torch.zeros_like(grad, dtype=torch.float64)
        want.index_add_(0, ids, gout.double())
        assert (grad.double() - want).abs().max().item() <= 1e-5
        if z is not None:
            got = grad.reshape(-1)[torch.from_numpy(z["grad_idx"]).to(cuda_device)]
            assert np.abs(got.double().cpu().numpy() - z["grad_val"]).max() <= 1e-5
        csrc.check_device_status()
    finally:
        tree.zero_grad(set_to_none=True)
        case["tree"].to("cpu")


@pytest.mark.parametrize("name", ["c3_full_image", "c5_full_image"])
def test_image_full_size(name, cuda_device):
    # One view of each forward benchmark at full resolution on the full tree; the second
    # tree holds more than 2^31 floats.
    from oracle import oracle as orc
    case = FULL_CASES[name]()
    z = _gold(name)
    cam = case["camera"]
    tree = case["tree"].to(cuda_device)
    try:
        if name == "c5_full_image":
            assert tree.data.numel() > 2 ** 31
        r = P._renderer(tree, case)
        with torch.no_grad():
            img = r.render_persp(cam["c2w"].to(cuda_device), width=cam["width"],
                                 height=cam["height"], fx=cam["fx"], fy=cam["fy"],
                                 fast=case["fast"])
            with r.frozen_tree():                   # the index kept by the caller: same image
                again = r.render_persp(cam["c2w"].to(cuda_device), width=cam["width"],
                                       height=cam["height"], fx=cam["fx"], fy=cam["fy"],
                                       fast=case["fast"])
        assert torch.equal(img, again)
        csrc.check_device_status()
        flat = img.reshape(-1, 3).cpu().numpy()
        if z is not None:
            assert np.abs(flat[::FULL_PIXEL_STRIDE] - z["out"]).max() <= RGB_TOL
        # the oracle on a seeded sample of the pixels (all of them would take minutes)
        case["tree"].to("cpu")
        o, d = orc.pixel_rays(cam["c2w"].numpy(), cam["fx"], cam["fy"], cam["width"],
                              cam["height"])
        pick = np.sort(np.random.default_rng(5).choice(o.shape[0], 40000, replace=False))
        ot = orc.Tree.from_n3tree(case["tree"])
        want = orc.volume_render(ot, o[pick], d[pick], d[pick], P._oracle_options(case))
        assert np.abs(flat[pick] - want).max() <= RGB_TOL
        assert (np.abs(want - 1.0).max(axis=1) > 1e-3).mean() > 0.02   # the sample sees the scene
    finally:
        case["tree"].to("cpu")


def test_image_backward_full_size(cuda_device):
    # The 800x800 view of the 512^3 shell tree (SH16, K = 49) with gradients: logged forward and
    # replay backward over pixel rays at full size, against the reference's
    # volume_render_image[_backward] and the oracle.
    case = FULL_CASES["c3_full_image_grad"]()
    z = _gold("c3_full_image_grad")
    assert z is not None
    mine = P.run_product(case, cuda_device)
    flat = mine["out"].reshape(-1, 3)
    assert np.abs(flat[::FULL_PIXEL_STRIDE] - z["out"]).max() <= RGB_TOL
    orc = P.run_oracle(case)
    assert np.abs(mine["out"] - orc["out"]).max() <= RGB_TOL
    idx = z["grad_idx"]
    scale = orc["grad_abs"].reshape(-1)[idx]
    P.assert_grad_matches_reference(mine["grad"].reshape(-1)[idx], z["grad_val"], scale,
                                    "image backward")
    assert P.grad_excess(mine["grad"], orc["grad"], orc["grad_abs"], 1e-3) <= 1.0
    total = float(z["grad_abs_sum"])
    assert abs(np.abs(mine["grad"]).sum() - total) <= 1e-5 * total
    march = P.run_product(case, cuda_device, item_log=False)
    P.assert_grad_matches_reference(march["grad"].reshape(-1)[idx], z["grad_val"], scale,
                                    "marching image backward")
