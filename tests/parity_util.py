"""Run one parity case (tests/golden/cases.py) through each implementation.

* ``run_product``  -- the CUDA path of svox_b200, through its public API
* ``run_oracle``   -- the CPU oracle (oracle/)
* ``run_ref_cuda`` -- the unmodified reference extension built into
  ``oracle/_ref`` (GPU only; used to generate fixtures and as an extra check)

Each returns a dict with ``out`` (rendered colours or queried values),
``ids`` (query) and ``grad`` (gradient w.r.t. tree.data, float64 numpy or
None).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QUERY_ROWS_KEPT = 256  # query fixtures keep the values of this many points

import svox_b200  # noqa: E402
from svox_b200 import csrc as _C  # noqa: E402


def _renderer(tree, case):
    r = svox_b200.VolumeRenderer(tree, **case["render"])
    for k, v in case["attrs"].items():
        setattr(r, k, v)
    return r


def options_of(case):
    """The RenderOptions the renderer would pack for this case."""
    return _renderer(case["tree"], case)._get_options(case["fast"])


# ---------------------------------------------------------------------------
def run_product(case, device="cuda:0", backward=True, single_march=True, item_log=True):
    """``item_log=False`` makes the backward march the rays (one march if
    ``single_march``) instead of replaying the forward's item log."""
    from svox_b200 import render as _render
    _render.USE_ITEM_LOG = bool(item_log)
    _render.FORCE_TWO_MARCHES = not single_march
    try:
        return _run_product(case, device, backward, single_march)
    finally:
        _render.USE_ITEM_LOG = True
        _render.FORCE_TWO_MARCHES = False


def _run_product(case, device, backward, single_march):
    tree = case["tree"].to(device)
    tree.zero_grad(set_to_none=True)
    res = {"ids": None, "grad": None}
    if case["kind"] == "query":
        pts = case["points"].to(device)
        vals, ids = tree(pts, want_node_ids=True)
        res["out"], res["ids"] = vals.detach().cpu().numpy(), ids.cpu().numpy()
        if backward and case["grad_out"] is not None:
            vals.backward(case["grad_out"].to(device))
    else:
        r = _renderer(tree, case)
        if case["kind"] == "rays":
            rays = svox_b200.Rays(*[t.to(device) for t in case["rays"]])
            out = r(rays, fast=case["fast"])
        else:
            cam = case["camera"]
            out = r.render_persp(cam["c2w"].to(device), width=cam["width"], height=cam["height"],
                                 fx=cam["fx"], fy=cam["fy"], fast=case["fast"])
        res["out"] = out.detach().cpu().numpy()
        if backward and case["mse_targets"] is not None:
            ((out - case["mse_targets"].to(device)) ** 2).mean().backward()
        elif backward and case["grad_out"] is not None:
            out.backward(case["grad_out"].to(device))
    if tree.data.grad is not None:
        res["grad"] = tree.data.grad.double().cpu().numpy()
    _C.check_device_status()
    case["tree"].to("cpu")
    tree.zero_grad(set_to_none=True)
    return res


# ---------------------------------------------------------------------------
def _oracle_options(case):
    from oracle import oracle as orc
    po = options_of(case)
    return orc.options(step_size=po.step_size, background_brightness=po.background_brightness,
                       format=po.format, basis_dim=po.basis_dim, ndc_width=po.ndc_width,
                       ndc_height=po.ndc_height, ndc_focal=po.ndc_focal, min_comp=po.min_comp,
                       max_comp=po.max_comp, sigma_thresh=po.sigma_thresh,
                       stop_thresh=po.stop_thresh, density_softplus=po.density_softplus,
                       rgb_padding=po.rgb_padding)


def _upstream(case, out):
    """The gradient that reaches the render's output: given, or that of the MSE loss."""
    if case["mse_targets"] is not None:
        tg = case["mse_targets"].numpy()
        return ((2.0 / out.size) * (out - tg)).astype(np.float32)
    return None if case["grad_out"] is None else case["grad_out"].numpy()


def run_oracle(case, backward=True, want_counts=False):
    """Also returns ``grad_abs``: per element the sum of |contributions|, the scale
    against which a sum formed by float atomics in any order may differ."""
    from oracle import oracle as orc
    tree = case["tree"]
    res = {"ids": None, "grad": None, "grad_abs": None}
    if case["kind"] == "query":
        ot = orc.Tree.from_n3tree(tree, world=True)
        pts = case["points"].numpy()
        res["out"], res["ids"] = orc.query_vertical(ot, pts)
        if backward and case["grad_out"] is not None:
            g = case["grad_out"].numpy()
            res["grad"] = orc.query_vertical_backward(ot, pts, g)
            res["grad_abs"] = orc.query_vertical_backward(ot, pts, np.abs(g))
        return res
    ot = orc.Tree.from_n3tree(tree, world=True)
    opt = _oracle_options(case)
    if case["kind"] == "rays":
        o, d, v = [t.numpy() for t in case["rays"]]
        r = orc.volume_render(ot, o, d, v, opt, want_counts=want_counts)
        if want_counts:
            res["out"], res["visits"], res["contrib"] = r
        else:
            res["out"] = r
        gout = _upstream(case, res["out"])
        if backward and gout is not None:
            res["grad"], res["grad_abs"] = orc.volume_render_backward(
                ot, o, d, v, opt, gout, want_abs=True)
    else:
        cam = case["camera"]
        args = (cam["c2w"].numpy(), cam["fx"], cam["fy"], cam["width"], cam["height"], opt)
        r = orc.volume_render_image(ot, *args, want_counts=want_counts)
        if want_counts:
            res["out"], res["visits"], res["contrib"] = r
        else:
            res["out"] = r
        if backward and case["grad_out"] is not None:
            res["grad"], res["grad_abs"] = orc.volume_render_image_backward(
                ot, *args, case["grad_out"].numpy(), want_abs=True)
    return res


# ---------------------------------------------------------------------------
_ref_mod = None


def ref_module():
    global _ref_mod
    if _ref_mod is None:
        from oracle.build_ref import load_module
        _ref_mod = load_module()
    return _ref_mod


def run_ref_cuda(case, device="cuda:0", backward=True, weight_op=None):
    """``weight_op`` ("sum" / "max"): forward only, with the reference's weight accumulator
    switched on; the flat accumulator comes back as ``weights``."""
    ref = ref_module()
    assert ref is not None, "oracle/_ref is not built"
    tree = case["tree"].to(device)
    spec = ref.TreeSpec()
    spec.data, spec.child, spec.parent_depth = tree.data.data, tree.child, tree.parent_depth
    spec.extra_data = tree.extra_data if tree.extra_data is not None else \
        torch.empty((0, 0), device=device)
    spec.offset, spec.scaling = tree.offset, tree.invradius
    spec._weight_accum = torch.empty(0, device=device)
    spec._weight_accum_max = False
    if weight_op is not None:
        spec._weight_accum = torch.zeros(tree.child.shape, device=device)
        spec._weight_accum_max = weight_op == "max"
        backward = False
    res = {"ids": None, "grad": None}
    if case["kind"] == "query":
        pts = case["points"].to(device)
        vals, ids = ref.query_vertical(spec, pts)
        res["out"], res["ids"] = vals.cpu().numpy(), ids.cpu().numpy()
        if backward and case["grad_out"] is not None:
            g = ref.query_vertical_backward(spec, pts, case["grad_out"].to(device))
            res["grad"] = g.double().cpu().numpy()
    else:
        po = options_of(case)
        opt = ref.RenderOptions()
        for k in ("step_size", "background_brightness", "format", "basis_dim", "ndc_width",
                  "ndc_height", "ndc_focal", "min_comp", "max_comp", "sigma_thresh",
                  "stop_thresh", "density_softplus", "rgb_padding"):
            setattr(opt, k, getattr(po, k))
        if case["kind"] == "rays":
            rs = ref.RaysSpec()
            rs.origins, rs.dirs, rs.vdirs = [t.to(device).contiguous() for t in case["rays"]]
            out = ref.volume_render(spec, rs, opt)
            res["out"] = out.cpu().numpy()
            gout = case["grad_out"]
            if case["mse_targets"] is not None:
                gout = (2.0 / out.numel()) * (out - case["mse_targets"].to(device))
            if backward and gout is not None:
                g = ref.volume_render_backward(spec, rs, opt, gout.to(device).contiguous())
                res["grad"] = g.double().cpu().numpy()
        else:
            cam = case["camera"]
            cs = ref.CameraSpec()
            cs.c2w = cam["c2w"].to(device).contiguous()
            cs.width, cs.height, cs.fx, cs.fy = cam["width"], cam["height"], cam["fx"], cam["fy"]
            out = ref.volume_render_image(spec, cs, opt)
            res["out"] = out.cpu().numpy()
            if backward and case["grad_out"] is not None:
                g = ref.volume_render_image_backward(spec, cs, opt, case["grad_out"].to(device))
                res["grad"] = g.double().cpu().numpy()
    torch.cuda.synchronize()
    if weight_op is not None:
        res["weights"] = spec._weight_accum.cpu().numpy().reshape(-1)
    case["tree"].to("cpu")
    return res


# ---------------------------------------------------------------------------
# Gradient fixtures: the full gradient is as large as the tree, so a fixture
# keeps a seeded sample of its non-zero elements plus two global sums.
def grad_digest(grad, n_sample=20000, seed=0):
    flat = np.asarray(grad, dtype=np.float64).reshape(-1)
    nz = np.flatnonzero(flat)
    rng = np.random.default_rng(seed)
    idx = np.sort(rng.choice(nz, size=min(n_sample, nz.size), replace=False)) if nz.size else nz
    return dict(grad_idx=idx.astype(np.int64), grad_val=flat[idx], grad_sum=flat.sum(),
                grad_abs_sum=np.abs(flat).sum(), grad_nnz=np.int64(nz.size),
                grad_max=np.abs(flat).max() if flat.size else 0.0)


def grad_excess(grad, ref_grad, grad_abs, rel_tol=1e-4):
    """Worst |g - ref| in units of the tolerance rel_tol * sum|contributions|
    (floored at 1e-4 of the largest gradient); <= 1 means within tolerance.  Used against the
    CPU oracle, whose libm expf differs from CUDA's in the last bit."""
    g, r = np.asarray(grad, np.float64).reshape(-1), np.asarray(ref_grad, np.float64).reshape(-1)
    scale = np.maximum(np.asarray(grad_abs, np.float64).reshape(-1), 1e-4 * np.abs(r).max())
    return float((np.abs(g - r) / (rel_tol * scale)).max())


# Gradient against the reference's CUDA extension.  Every gradient element is a sum of float
# atomics, so the reference does not even reproduce itself: two runs of it on the same inputs
# (fixtures: grad_val, grad_val2) differ by up to 2e-7 of an element's summed |contributions|,
# and where the contributions cancel that is far more than 1e-4 of the element's VALUE (the
# full-size training step: 6e-3 between the reference's own two runs).  So "within 1e-4
# relative" is asserted in the two forms that a float sum can meet:
#   * the whole gradient: max |g - ref| / max |ref| <= GRAD_MAXNORM_TOL (ten times tighter
#     than 1e-4; observed < 1e-6);
#   * every element: |g - ref| <= 1e-4 |ref| + GRAD_CANCEL_TOL * sum|contributions|.
#     Observed: < 7e-6 of the summed magnitude (the kernels also take the running sum of the
#     reference's second march from the forward's result, a few more roundings than a
#     reordering of atomics), the reference against itself 3e-7.
GRAD_MAXNORM_TOL = 1e-5
GRAD_REL_TOL = 1e-4
GRAD_CANCEL_TOL = 2e-5


def grad_deviation(grad, ref_grad, grad_abs):
    """-> (max-norm error, worst element in units of its allowance); both must be <= 1 after
    dividing the first by GRAD_MAXNORM_TOL."""
    g, r = np.asarray(grad, np.float64).reshape(-1), np.asarray(ref_grad, np.float64).reshape(-1)
    top = np.abs(r).max()
    if top == 0:
        return float(np.abs(g).max()), 0.0
    err = np.abs(g - r)
    allow = GRAD_REL_TOL * np.abs(r) + GRAD_CANCEL_TOL * np.maximum(
        np.asarray(grad_abs, np.float64).reshape(-1), 1e-4 * top)
    return float(err.max() / top), float((err / allow).max())


def assert_grad_matches_reference(grad, ref_grad, grad_abs, what="gradient"):
    maxnorm, worst = grad_deviation(grad, ref_grad, grad_abs)
    assert maxnorm <= GRAD_MAXNORM_TOL, f"{what}: max-norm error {maxnorm:.3g}"
    assert worst <= 1.0, f"{what}: an element is off by {worst:.2f} x its allowance"
    return maxnorm, worst


def grad_error(grad, ref_grad):
    """max |g - ref| / max |ref| and the worst element-wise relative error over elements with
    |ref| > 1e-6 * max|ref| (reported, not asserted: see above)."""
    g, r = np.asarray(grad, np.float64).reshape(-1), np.asarray(ref_grad, np.float64).reshape(-1)
    scale = np.abs(r).max()
    if scale == 0:
        return float(np.abs(g).max()), 0.0
    err = np.abs(g - r)
    big = np.abs(r) > 1e-6 * scale
    rel = float((err[big] / np.abs(r[big])).max()) if big.any() else 0.0
    return float(err.max() / scale), rel


def run_weight_accumulation(case, op, device=None):
    """Per-leaf weight accumulator of one forward render: product (``device`` given) or
    oracle (``device`` None), as a flat float64 array over (M, N, N, N)."""
    tree = case["tree"]
    if device is None:
        from oracle import oracle as orc
        ot = orc.Tree.from_n3tree(tree, world=True)
        opt = _oracle_options(case)
        with orc.weight_accumulation(ot, op) as acc:
            if case["kind"] == "rays":
                o, d, v = [t.numpy() for t in case["rays"]]
                orc.volume_render(ot, o, d, v, opt)
            else:
                cam = case["camera"]
                orc.volume_render_image(ot, cam["c2w"].numpy(), cam["fx"], cam["fy"],
                                        cam["width"], cam["height"], opt)
        return acc.reshape(-1).copy()
    t = tree.to(device)
    try:
        r = _renderer(t, case)
        with torch.no_grad(), t.accumulate_weights(op=op) as accum:
            if case["kind"] == "rays":
                r(svox_b200.Rays(*[x.to(device) for x in case["rays"]]), fast=case["fast"])
            else:
                cam = case["camera"]
                r.render_persp(cam["c2w"].to(device), width=cam["width"], height=cam["height"],
                               fx=cam["fx"], fy=cam["fy"], fast=case["fast"])
            dense = accum.value.double().cpu().numpy().reshape(-1)
            per_leaf = accum().double().cpu().numpy()
        _C.check_device_status()
        n = t.n_internal * t.N ** 3
        return dense[:n], per_leaf
    finally:
        case["tree"].to("cpu")


# ---------------------------------------------------------------------------
# se_grad: rendered colour, gradient and Gauss-Newton diagonal of the squared error

def se_grad_colors(case):
    """Seeded reference colours for a case: (Q, 3) for rays, (H, W, 3) for a camera."""
    gen = torch.Generator().manual_seed(977)
    if case["kind"] == "rays":
        return torch.rand(case["rays"][0].shape[0], 3, generator=gen)
    cam = case["camera"]
    return torch.rand(cam["height"], cam["width"], 3, generator=gen)


def run_se_grad(case, which, device="cuda:0"):
    """``which``: "product", "oracle" or "ref_cuda" -> dict(out, grad, hess[, grad_abs])."""
    tree = case["tree"]
    colors = se_grad_colors(case)
    if which == "oracle":
        from oracle import oracle as orc
        ot = orc.Tree.from_n3tree(tree, world=True)
        opt = _oracle_options(case)
        if case["kind"] == "rays":
            o, d, v = [t.numpy() for t in case["rays"]]
        else:
            cam = case["camera"]
            o, d = orc.pixel_rays(cam["c2w"].numpy(), cam["fx"], cam["fy"], cam["width"],
                                  cam["height"])
            v = d
        out, grad, hess, gabs = orc.se_grad(ot, o, d, v, opt, colors.reshape(-1, 3).numpy(),
                                            want_abs=True)
        return dict(out=out.reshape(colors.shape), grad=grad, hess=hess, grad_abs=gabs)
    t = tree.to(device)
    try:
        if which == "product":
            r = _renderer(t, case)
            if case["kind"] == "rays":
                res = r.se_grad(svox_b200.Rays(*[x.to(device) for x in case["rays"]]),
                                colors.to(device))
            else:
                cam = case["camera"]
                res = r.se_grad_persp(cam["c2w"].to(device), colors.to(device),
                                      width=cam["width"], height=cam["height"], fx=cam["fx"],
                                      fy=cam["fy"])
            _C.check_device_status()
        else:
            ref = ref_module()
            assert ref is not None, "oracle/_ref is not built"
            spec = ref.TreeSpec()
            spec.data, spec.child, spec.parent_depth = t.data.data, t.child, t.parent_depth
            spec.extra_data = t.extra_data if t.extra_data is not None else \
                torch.empty((0, 0), device=device)
            spec.offset, spec.scaling = t.offset, t.invradius
            spec._weight_accum = torch.empty(0, device=device)
            spec._weight_accum_max = False
            po = options_of(case)
            opt = ref.RenderOptions()
            for k in ("step_size", "background_brightness", "format", "basis_dim", "ndc_width",
                      "ndc_height", "ndc_focal", "min_comp", "max_comp", "sigma_thresh",
                      "stop_thresh", "density_softplus", "rgb_padding"):
                setattr(opt, k, getattr(po, k))
            if case["kind"] == "rays":
                rs = ref.RaysSpec()
                rs.origins, rs.dirs, rs.vdirs = [x.to(device).contiguous() for x in case["rays"]]
                res = ref.se_grad(spec, rs, colors.to(device), opt)
            else:
                cam = case["camera"]
                cs = ref.CameraSpec()
                cs.c2w = cam["c2w"].to(device).contiguous()
                cs.width, cs.height, cs.fx, cs.fy = (cam["width"], cam["height"], cam["fx"],
                                                     cam["fy"])
                res = ref.se_grad_persp(spec, cs, opt, colors.to(device))
            torch.cuda.synchronize()
        out, grad, hess = res
        return dict(out=out.cpu().numpy(), grad=grad.double().cpu().numpy(),
                    hess=hess.double().cpu().numpy())
    finally:
        case["tree"].to("cpu")
