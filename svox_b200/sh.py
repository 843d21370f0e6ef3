"""Real spherical-harmonic basis in tensor ops (``svox.sh``: ``eval_sh_bases``, ``eval_sh``).

The kernels evaluate the same polynomials on the device (``sh_basis`` in
``svox_b200/csrc/render.cuh``); this module is the host-side counterpart for code that wants the
basis as a tensor, e.g. to turn SH coefficients into colours for given view directions.  Basis
function k of degree l, order m sits at index ``l * l + l + m``; the normalisation and the signs
are those of the reference (svox/sh.py:27-161), so coefficients trained against one are valid for
the other.
"""
import torch

__all__ = ["eval_sh_bases", "eval_sh"]

_C0 = 0.28209479177387814
_C1 = 0.4886025119029199
_C2 = (1.0925484305920792, -1.0925484305920792, 0.31539156525252005, -1.0925484305920792,
       0.5462742152960396)
_C3 = (-0.5900435899266435, 2.890611442640554, -0.4570457994644658, 0.3731763325901154,
       -0.4570457994644658, 1.445305721320277, -0.5900435899266435)
_C4 = (2.5033429417967046, -1.7701307697799304, 0.9461746957575601, -0.6690465435572892,
       0.10578554691520431, -0.6690465435572892, 0.47308734787878004, -1.7701307697799304,
       0.6258357354491761)


def eval_sh_bases(deg, dirs):
    """``(..., 3)`` unit directions -> ``(..., (deg + 1) ** 2)`` basis values, ``0 <= deg <= 4``."""
    assert 0 <= deg <= 4
    x, y, z = dirs[..., 0], dirs[..., 1], dirs[..., 2]
    cols = [torch.full_like(x, _C0)]
    if deg >= 1:
        cols += [-_C1 * y, _C1 * z, -_C1 * x]
    if deg >= 2:
        xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
        cols += [_C2[0] * xy, _C2[1] * yz, _C2[2] * (2.0 * zz - xx - yy), _C2[3] * xz,
                 _C2[4] * (xx - yy)]
    if deg >= 3:
        cols += [_C3[0] * y * (3 * xx - yy), _C3[1] * xy * z, _C3[2] * y * (4 * zz - xx - yy),
                 _C3[3] * z * (2 * zz - 3 * xx - 3 * yy), _C3[4] * x * (4 * zz - xx - yy),
                 _C3[5] * z * (xx - yy), _C3[6] * x * (xx - 3 * yy)]
    if deg >= 4:
        cols += [_C4[0] * xy * (xx - yy), _C4[1] * yz * (3 * xx - yy), _C4[2] * xy * (7 * zz - 1),
                 _C4[3] * yz * (7 * zz - 3), _C4[4] * (zz * (35 * zz - 30) + 3),
                 _C4[5] * xz * (7 * zz - 3), _C4[6] * (xx - yy) * (7 * zz - 1),
                 _C4[7] * xz * (xx - 3 * yy),
                 _C4[8] * (xx * (xx - 3 * yy) - yy * (3 * xx - yy))]
    return torch.stack(cols, dim=-1)


def eval_sh(deg, sh, dirs):
    """Coefficients ``sh (..., C, (deg + 1) ** 2)`` at directions ``dirs (..., 3)`` ->
    ``(..., C)``: the basis-weighted sum per channel."""
    assert sh.shape[-1] >= (deg + 1) ** 2
    basis = eval_sh_bases(deg, dirs)
    return (sh[..., :basis.shape[-1]] * basis[..., None, :]).sum(dim=-1)
