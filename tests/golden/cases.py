"""Seeded parity cases shared by the fixture generators and the tests.

Every case is rebuilt from its seed on the CPU (trees and inputs are not
stored); the fixtures under this directory only hold the OUTPUTS that the
reference produced for them.  Each builder returns a dict:

    tree     svox_b200.N3Tree on the CPU
    kind     "rays" | "image" | "query"
    rays     svox_b200.Rays            (kind == "rays")
    grad_out upstream gradient         (rays / image; None -> no backward)
    mse_targets  instead of grad_out: colours (Q, 3); the loss is the mean squared error
                 against them, so the upstream gradient is 2 (out - targets) / (3 Q)
    camera   dict(c2w, width, height, fx, fy)   (kind == "image")
    points   (Q, 3) world points, grad_out (Q, K)  (kind == "query")
    render   kwargs for VolumeRenderer(tree, **render)
    attrs    attributes set on the renderer (sigma_thresh / stop_thresh overrides)
    fast     the ``fast`` flag of the render call
"""
import torch

from svox_b200 import N3Tree, NDCConfig, Rays
from svox_b200 import workloads as W


def _g(seed):
    return torch.Generator().manual_seed(seed)


def _unit(v):
    return v / v.norm(dim=-1, keepdim=True)


def _small_shell(fmt, seed, init_refine=3, extra=3):
    gen = _g(seed)
    tree = W.shell_tree(init_refine, extra, fmt, gen, (5.0, 50.0),
                        [((0.5, 0.5, 0.5), 0.30, 0.35)])
    return tree, gen


def _base(tree, kind, **kw):
    d = dict(tree=tree, kind=kind, render={}, attrs={}, fast=False, grad_out=None,
             mse_targets=None)
    d.update(kw)
    return d


def c1_rays():
    """Smoke configuration: 16^3-leaf SH4 tree, 4096 rays, backward of sum(rgb)."""
    tree, rays = W.config1()
    return _base(tree, "rays", rays=rays, grad_out=torch.ones(rays.origins.shape[0], 3))


def shell_sh9_rays():
    """Config-4-like scene at 1/4 resolution: shell refined to 128^3, SH9, 8192 rays."""
    tree, gen = _small_shell("SH9", 103)
    rays = W.sphere_rays(8192, gen, 4.0, 0.2, 0.8)
    gout = torch.randn(8192, 3, generator=gen)
    return _base(tree, "rays", rays=rays, grad_out=gout)


def c4_sample_rays():
    """The training-step benchmark scene (full 512^3 shell tree), first 16384 rays of its 2^20,
    forward only."""
    tree, rays, _ = W.config4(Q=1 << 14)
    return _base(tree, "rays", rays=rays)


def shell_sh16_image():
    """Config-3-like scene at 1/4 resolution: SH16, 96x96 image, stop_thresh 1e-2."""
    tree, gen = _small_shell("SH16", 102)
    c2w = W.look_at_cameras(1, gen, 4.0)[0]
    gout = torch.randn(96, 96, 3, generator=gen)
    return _base(tree, "image", camera=dict(c2w=c2w, width=96, height=96, fx=133.0, fy=133.0),
                 attrs=dict(stop_thresh=1e-2), grad_out=gout)


def _variant(seed=104, Q=2048, **kw):
    tree, gen = _small_shell("SH9", seed, extra=2)
    rays = W.sphere_rays(Q, gen, 4.0, 0.2, 0.8)
    gout = torch.randn(Q, 3, generator=gen)
    return _base(tree, "rays", rays=rays, grad_out=gout, **kw)


def opt_fast():
    """fast=True: sigma_thresh = stop_thresh = 1e-2."""
    return _variant(fast=True)


def opt_softplus_pad_bg():
    """density_softplus, rgb_padding, grey background, smaller step."""
    return _variant(render=dict(density_softplus=True, rgb_padding=0.001,
                                background_brightness=0.5, step_size=5e-4))


def opt_comp_range():
    """Only SH components 1..3 are rendered."""
    return _variant(render=dict(min_comp=1, max_comp=3))


def rgba_rays():
    """RGBA records (K = 4), uniform 8^3 tree."""
    gen = _g(105)
    tree = W.uniform_tree(2, "RGBA", gen, sigma_range=(0.0, 20.0))
    rays = W.sphere_rays(1024, gen, 2.0, 0.3, 0.7)
    return _base(tree, "rays", rays=rays, grad_out=torch.randn(1024, 3, generator=gen))


def sh1_rays():
    gen = _g(106)
    tree = W.uniform_tree(2, "SH1", gen, sigma_range=(0.0, 20.0))
    rays = W.sphere_rays(1024, gen, 2.0, 0.3, 0.7)
    return _base(tree, "rays", rays=rays, grad_out=torch.randn(1024, 3, generator=gen))


def sh25_rays():
    gen = _g(107)
    tree = W.uniform_tree(2, "SH25", gen, sigma_range=(0.0, 20.0), coef_std=0.5)
    rays = W.sphere_rays(1024, gen, 2.0, 0.3, 0.7)
    return _base(tree, "rays", rays=rays, grad_out=torch.randn(1024, 3, generator=gen))


def _lobes(gen, n, anisotropic):
    """Seeded lobe parameters (the tree's ``extra_data``): SG rows are [sharpness, axis xyz];
    ASG rows are [bandwidth x, bandwidth y, frame x axis, y axis, z axis], the frame orthonormal."""
    z = _unit(torch.randn(n, 3, generator=gen))
    if not anisotropic:
        return torch.cat([0.5 + 4.0 * torch.rand(n, 1, generator=gen), z], dim=1)
    a = torch.randn(n, 3, generator=gen)
    x = _unit(a - (a * z).sum(-1, keepdim=True) * z)
    y = torch.cross(z, x, dim=-1)
    return torch.cat([0.5 + 4.0 * torch.rand(n, 2, generator=gen), x, y, z], dim=1)


def _lobe_case(fmt, seed, anisotropic, basis_dim, **kw):
    gen = _g(seed)
    tree = W.shell_tree(3, 2, f"{fmt}{basis_dim}", gen, (5.0, 50.0),
                        [((0.5, 0.5, 0.5), 0.30, 0.35)], coef_std=3.0,
                        extra_data=_lobes(gen, basis_dim, anisotropic))
    rays = W.sphere_rays(2048, gen, 4.0, 0.2, 0.8)
    return _base(tree, "rays", rays=rays, grad_out=torch.randn(2048, 3, generator=gen), **kw)


def sg9_rays():
    """Spherical-Gaussian colour, 9 lobes: a basis size the specialised kernels cover."""
    return _lobe_case("SG", 115, False, 9)


def sg5_rays():
    """Spherical-Gaussian colour, 5 lobes (no specialised kernel), components 1..3 only."""
    return _lobe_case("SG", 116, False, 5, render=dict(min_comp=1, max_comp=3))


def asg4_rays():
    """Anisotropic spherical-Gaussian colour, 4 lobes, density_softplus."""
    return _lobe_case("ASG", 117, True, 4, render=dict(density_softplus=True))


def asg7_image():
    """Anisotropic spherical-Gaussian colour, 7 lobes, perspective image."""
    gen = _g(118)
    tree = W.shell_tree(3, 2, "ASG7", gen, (5.0, 50.0), [((0.5, 0.5, 0.5), 0.30, 0.35)],
                        coef_std=3.0, extra_data=_lobes(gen, 7, True))
    c2w = W.look_at_cameras(1, gen, 4.0)[0]
    return _base(tree, "image", camera=dict(c2w=c2w, width=64, height=64, fx=200.0, fy=210.0),
                 grad_out=torch.randn(64, 64, 3, generator=gen))


def _aniso_tree(gen, fmt="SH4"):
    tree = N3Tree(N=2, data_format=fmt, init_refine=2, radius=[0.6, 0.8, 1.0],
                  center=[0.1, -0.2, 0.3])
    # irregular structure: refine a random third of the leaves twice
    for _ in range(2):
        mask = torch.rand(tree.n_leaves, generator=gen) < 0.33
        tree[mask].refine()
    with torch.no_grad():
        d = tree.data.data
        d[..., :-1] = torch.randn(d[..., :-1].shape, generator=gen)
        d[..., -1] = torch.rand(d[..., -1].shape, generator=gen) * 12.0 - 2.0
    return tree


def aniso_rays():
    """Non-cubic world box (scaling != 1, offset != 0), irregular depth, negative densities."""
    gen = _g(108)
    tree = _aniso_tree(gen)
    Q = 2048
    origins = torch.tensor([0.1, -0.2, 0.3]) + 3.0 * _unit(torch.randn(Q, 3, generator=gen))
    targets = torch.tensor([0.1, -0.2, 0.3]) + (torch.rand(Q, 3, generator=gen) - 0.5) * \
        torch.tensor([1.0, 1.4, 1.8])
    dirs = _unit(targets - origins) * (0.5 + torch.rand(Q, 1, generator=gen))  # non-unit dirs
    vdirs = _unit(dirs + 0.05 * torch.randn(Q, 3, generator=gen))
    return _base(tree, "rays", rays=Rays(origins, dirs, vdirs),
                 grad_out=torch.randn(Q, 3, generator=gen))


def aniso_image():
    """Perspective image of the non-cubic, irregular tree (image kernels' world transform)."""
    gen = _g(114)
    tree = _aniso_tree(gen)
    c2w = W.look_at_cameras(1, gen, 3.0, center=0.0)[0]
    c2w[:, 3] += torch.tensor([0.1, -0.2, 0.3])
    return _base(tree, "image", camera=dict(c2w=c2w, width=80, height=60, fx=70.0, fy=75.0),
                 grad_out=torch.randn(60, 80, 3, generator=gen))


def ndc_image():
    """Forward-facing camera rendered through the NDC warp; world box [-1,1]^3."""
    gen = _g(109)
    tree = N3Tree(N=2, data_format="SH4", init_refine=3, radius=1.0, center=[0.0, 0.0, 0.0])
    with torch.no_grad():
        d = tree.data.data
        d[..., :-1] = torch.randn(d[..., :-1].shape, generator=gen)
        d[..., -1] = torch.rand(d[..., -1].shape, generator=gen) * 6.0
    c2w = torch.tensor([[0.9950, 0.0, 0.0998, 0.10],
                        [0.0050, 0.9987, -0.0498, -0.05],
                        [-0.0997, 0.0500, 0.9938, 0.20]])
    return _base(tree, "image", camera=dict(c2w=c2w, width=64, height=48, fx=60.0, fy=60.0),
                 render=dict(ndc=NDCConfig(width=64, height=48, focal=60.0)),
                 grad_out=torch.randn(48, 64, 3, generator=gen))


def n3_rays():
    """Branching factor 3 (27 children per node)."""
    gen = _g(110)
    tree = N3Tree(N=3, data_format="SH4", init_refine=2)
    with torch.no_grad():
        d = tree.data.data
        d[..., :-1] = torch.randn(d[..., :-1].shape, generator=gen)
        d[..., -1] = torch.rand(d[..., -1].shape, generator=gen) * 10.0
    rays = W.sphere_rays(1024, gen, 2.0, 0.3, 0.7)
    return _base(tree, "rays", rays=rays, grad_out=torch.randn(1024, 3, generator=gen))


def _edge_points(gen, Q, lo, hi):
    """Uniform points plus the corner cases: cube faces, corners, outside, cell boundaries."""
    pts = torch.rand(Q, 3, generator=gen) * (hi - lo) + lo
    special = torch.tensor([[0.0, 0.0, 0.0], [1.0, 1.0, 1.0], [0.5, 0.5, 0.5], [-3.0, 0.2, 7.0],
                            [0.999999, 0.9999999, 1.0000001], [0.25, 0.75, 0.125],
                            [0.0625, 0.5, 0.99], [1e-9, 1e-20, 0.3]])
    special = special * (hi - lo) + lo
    pts[:special.shape[0]] = special
    return pts


def query_c1():
    """Point query on the config-1 tree incl. boundary and out-of-range points."""
    tree, _ = W.config1()
    gen = _g(111)
    pts = _edge_points(gen, 16384, torch.zeros(3), torch.ones(3))
    return _base(tree, "query", points=pts,
                 grad_out=torch.randn(16384, tree.data_dim, generator=gen))


def query_aniso():
    """Point query with a world transform on an irregular tree."""
    gen = _g(112)
    tree = _aniso_tree(gen, "SH9")
    lo = torch.tensor([0.1 - 0.6, -0.2 - 0.8, 0.3 - 1.0])
    hi = torch.tensor([0.1 + 0.6, -0.2 + 0.8, 0.3 + 1.0])
    pts = _edge_points(gen, 8192, lo, hi)
    return _base(tree, "query", points=pts,
                 grad_out=torch.randn(8192, tree.data_dim, generator=gen))


def query_shell():
    """Point query on the deep shell tree (depths 4..7 mixed)."""
    tree, gen = _small_shell("SH16", 113)
    pts = _edge_points(gen, 16384, torch.zeros(3), torch.ones(3))
    return _base(tree, "query", points=pts,
                 grad_out=torch.randn(16384, tree.data_dim, generator=gen))


CASES = {f.__name__: f for f in [
    c1_rays, shell_sh9_rays, c4_sample_rays, shell_sh16_image, opt_fast, opt_softplus_pad_bg,
    opt_comp_range, rgba_rays, sh1_rays, sh25_rays, aniso_rays, aniso_image, ndc_image, n3_rays,
    query_c1, query_aniso, query_shell, sg9_rays, sg5_rays, asg4_rays, asg7_image]}



def deep_rays():
    """A thin region refined to depth 10 around one point of a coarse tree: leaves far below the
    leaf table and its bricks, and leaves of every depth in between.  Oracle only (no fixture)."""
    gen = _g(120)
    tree = N3Tree(N=2, data_format="SH4", init_refine=1)
    p0 = torch.tensor([0.371, 0.412, 0.455])
    for k in range(8):
        centers = W._leaf_centers(tree)
        mask = (centers - p0).abs().max(dim=-1).values < 0.6 * 0.5 ** (k + 2)
        tree[mask].refine()
    with torch.no_grad():
        d = tree.data.data
        d[..., :-1] = torch.randn(d[..., :-1].shape, generator=gen)
        sig = torch.rand(d[..., -1].shape, generator=gen) * 40.0
        sig[torch.rand(sig.shape, generator=gen) < 0.3] = 0.0
        d[..., -1] = sig
    Q = 4096
    origins = 0.5 + 3.0 * _unit(torch.randn(Q, 3, generator=gen))
    targets = p0 + (torch.rand(Q, 3, generator=gen) - 0.5) * 0.02
    targets[Q // 2:] = 0.2 + 0.6 * torch.rand(Q - Q // 2, 3, generator=gen)
    dirs = _unit(targets - origins)
    return _base(tree, "rays", rays=Rays(origins, dirs, dirs),
                 grad_out=torch.randn(Q, 3, generator=gen))


# Cases without a reference fixture: checked against the oracle only.
EXTRA_CASES = {f.__name__: f for f in [deep_rays]}

def c4_full_rays():
    """The training-step benchmark itself: the full 512^3 shell tree, all 2^20 rays, gradient
    of the mean squared error against the seeded colour targets."""
    tree, rays, targets = W.config4()
    return _base(tree, "rays", rays=rays, mse_targets=targets)


def c2_full_query():
    """The query benchmark itself: uniform tree of 256^3 leaves, SH16 (3.76 GB of data, byte
    offsets beyond 2^31), 2^24 uniform points, N(0,1) upstream gradient."""
    tree, pts = W.config2()
    gout = torch.randn(pts.shape[0], tree.data_dim, generator=_g(121))
    return _base(tree, "query", points=pts, grad_out=gout)


def _full_view(cfg, width, height, focal, **kw):
    tree, cams = cfg(n_views=1)
    return _base(tree, "image", camera=dict(c2w=cams[0], width=width, height=height, fx=focal,
                                            fy=focal), **kw)


def c3_full_image():
    """First view of the sparse-shell forward benchmark: 512^3 shell, SH16, 800x800,
    stop_thresh 1e-2."""
    return _full_view(W.config3, 800, 800, 1111.0, attrs=dict(stop_thresh=1e-2))


def c3_full_image_grad():
    """The same 800x800 view without thresholds and with a seeded N(0,1) upstream gradient:
    the image backward (logged forward + replay backward over pixel rays) at full size."""
    case = _full_view(W.config3, 800, 800, 1111.0)
    case["grad_out"] = torch.randn(800, 800, 3, generator=_g(122))
    return case


def c5_full_image():
    """First view of the large multi-view benchmark: three shells refined to 1024^3, SH16
    (12 GB of data, element offsets beyond 2^31), 1920x1080, step 5e-4, fast=True."""
    return _full_view(W.config5, 1920, 1080, 1600.0, render=dict(step_size=5e-4), fast=True)


# Full-size cases: minutes of CPU work for the oracle, GPU tests only.  Their fixtures keep a
# strided sample of the outputs: the colours of every FULL_OUT_STRIDE-th ray, every
# FULL_PIXEL_STRIDE-th pixel (row-major), the leaf ids of every FULL_ID_STRIDE-th point.
FULL_CASES = {f.__name__: f for f in [c4_full_rays, c2_full_query, c3_full_image,
                                      c5_full_image, c3_full_image_grad]}
FULL_OUT_STRIDE = 16
FULL_PIXEL_STRIDE = 97
FULL_ID_STRIDE = 4096

# Cases whose fixtures are cheap enough to check on the CPU in the default test run.
BIG = {"c4_sample_rays"}
