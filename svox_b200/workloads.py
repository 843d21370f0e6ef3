"""Seeded synthetic scenes, rays and cameras used by the benchmark and the tests.

Real PlenOctree scenes are not available offline, so every workload is
drawn on the CPU from ``torch.Generator().manual_seed(seed)`` in a fixed
order (documented per function) and then moved to the device: every process
and every GPU sees identical bits.
"""
import math

import torch

from .render import Rays
from .tree import N3Tree

__all__ = ["uniform_tree", "shell_tree", "sphere_rays", "look_at_cameras",
           "config1", "config2", "config3", "config4", "config5"]


def _unit(v):
    return v / v.norm(dim=-1, keepdim=True)


def uniform_tree(init_refine, data_format, gen, sigma_range=None, coef_std=1.0):
    """Uniform tree with (2^(init_refine+1))^3 leaves.

    Draw order: all colour coefficients ~ N(0, coef_std), then (if
    ``sigma_range``) the density column ~ U[lo, hi]; otherwise the density
    column is N(0, coef_std) like the rest.
    """
    tree = N3Tree(N=2, data_format=data_format, init_refine=init_refine)
    with torch.no_grad():
        d = tree.data.data
        if sigma_range is None:
            d.copy_(torch.randn(d.shape, generator=gen) * coef_std)
        else:
            d[..., :-1] = torch.randn(d[..., :-1].shape, generator=gen) * coef_std
            lo, hi = sigma_range
            d[..., -1] = torch.rand(d[..., -1].shape, generator=gen) * (hi - lo) + lo
    return tree


def _leaf_centers(tree):
    view = tree[:]
    return view.corners_local + 0.5 * view.lengths_local[:, None]


def shell_tree(init_refine, extra_levels, data_format, gen, sigma_range, shells, coef_std=0.5,
               extra_data=None):
    """Uniform tree refined ``extra_levels`` more inside spherical shells.

    ``shells`` is a list of (centre(3), r_lo, r_hi).  A leaf of the uniform
    tree is selected when its centre lies in any shell; selected leaves are
    refined ``extra_levels`` times.  A final leaf is "in the shell" iff it is
    at the finest level and its own centre lies in a shell.  Draw order:
    colour coefficients ~ N(0, coef_std) for the whole data tensor, then one
    U[lo, hi] density per in-shell leaf in leaf order; all other densities 0.
    """
    tree = N3Tree(N=2, data_format=data_format, init_refine=init_refine, extra_data=extra_data)

    def in_any(centers):
        m = torch.zeros(centers.shape[0], dtype=torch.bool)
        for c, lo, hi in shells:
            dist = (centers - torch.as_tensor(c, dtype=centers.dtype)).norm(dim=1)
            m |= (dist >= lo) & (dist <= hi)
        return m

    tree[in_any(_leaf_centers(tree))].refine(extra_levels)
    with torch.no_grad():
        d = tree.data.data
        d[..., :-1] = torch.randn(d[..., :-1].shape, generator=gen) * coef_std
        d[..., -1] = 0.0
        view = tree[:]
        inside = in_any(_leaf_centers(tree)) & (view.depths.cpu() == init_refine + extra_levels)
        lo, hi = sigma_range
        sig = torch.rand(int(inside.sum()), generator=gen) * (hi - lo) + lo
        leaves = tree._all_leaves()[inside]
        d[leaves[:, 0], leaves[:, 1], leaves[:, 2], leaves[:, 3], -1] = sig
    return tree


def sphere_rays(Q, gen, radius, target_lo, target_hi, center=0.5):
    """Origins on a sphere, directions towards uniform targets; viewdirs = dirs.

    Draw order: origins N(0,1)^3 (normalised, scaled), then targets U[lo,hi]^3.
    """
    origins = center + radius * _unit(torch.randn(Q, 3, generator=gen))
    targets = torch.rand(Q, 3, generator=gen) * (target_hi - target_lo) + target_lo
    dirs = _unit(targets - origins)
    return Rays(origins=origins, dirs=dirs, viewdirs=dirs.clone())


def look_at_cameras(n, gen, radius, center=0.5):
    """``n`` camera-to-world (3,4) matrices on a sphere looking at the centre.

    OpenGL convention (camera looks down -z, y up); world up is +z, or +y
    when the view axis is parallel to it.
    """
    pos = center + radius * _unit(torch.randn(n, 3, generator=gen))
    out = []
    for p in pos:
        fwd = _unit(torch.full((3,), float(center)) - p)
        up = torch.tensor([0.0, 0.0, 1.0])
        if abs(float(fwd @ up)) > 0.999:
            up = torch.tensor([0.0, 1.0, 0.0])
        right = _unit(torch.linalg.cross(fwd, up))
        true_up = torch.linalg.cross(right, fwd)
        out.append(torch.stack([right, true_up, -fwd, p], dim=1))
    return torch.stack(out)


# ---------------------------------------------------------------------------
# The five benchmark configurations

def config1():
    """4096-leaf SH-degree-1 tree, 4096 rays from a radius-2 sphere (seed 0)."""
    gen = torch.Generator().manual_seed(0)
    tree = uniform_tree(3, "SH4", gen, sigma_range=(0.0, 10.0))
    Q = 4096
    origins = 0.5 + 2.0 * _unit(torch.randn(Q, 3, generator=gen))
    jitter = torch.rand(Q, 3, generator=gen) * 0.4 - 0.2
    dirs = _unit(0.5 + jitter - origins)
    return tree, Rays(origins, dirs, dirs.clone())


def config2(Q=1 << 24, init_refine=7):
    """256^3-leaf SH-degree-3 tree and Q uniform query points (seed 1)."""
    gen = torch.Generator().manual_seed(1)
    tree = uniform_tree(init_refine, "SH16", gen)
    points = torch.rand(Q, 3, generator=gen)
    return tree, points


_SHELL = [((0.5, 0.5, 0.5), 0.30, 0.35)]


def config3(n_views=8, init_refine=5, extra_levels=3):
    """Sparse-shell SH-degree-3 tree and 8 cameras on a radius-4 sphere (seed 2)."""
    gen = torch.Generator().manual_seed(2)
    tree = shell_tree(init_refine, extra_levels, "SH16", gen, (5.0, 50.0), _SHELL)
    cams = look_at_cameras(n_views, gen, 4.0)
    return tree, cams


def config4(Q=1 << 20, init_refine=5, extra_levels=3):
    """Sparse-shell SH-degree-2 tree, Q training rays and colour targets (seed 3)."""
    gen = torch.Generator().manual_seed(3)
    tree = shell_tree(init_refine, extra_levels, "SH9", gen, (5.0, 50.0), _SHELL)
    rays = sphere_rays(Q, gen, 4.0, 0.2, 0.8)
    targets = torch.rand(Q, 3, generator=gen)
    return tree, rays, targets


def config5(n_views=64, init_refine=6, extra_levels=3):
    """Three random shells refined to 1024^3, SH degree 3, 64 cameras (seed 4)."""
    gen = torch.Generator().manual_seed(4)
    shells = []
    for _ in range(3):
        c = (torch.rand(3, generator=gen) * 0.4 + 0.3).tolist()
        r = float(torch.rand(1, generator=gen) * 0.2 + 0.1)
        shells.append((tuple(c), r - 0.015, r + 0.015))
    tree = shell_tree(init_refine, extra_levels, "SH16", gen, (5.0, 100.0), shells)
    cams = look_at_cameras(n_views, gen, 3.0)
    return tree, cams
