"""Host logic: format parsing and render-option packing (no GPU)."""
import pytest
import torch

import svox_b200 as svox
from svox_b200 import DataFormat


@pytest.mark.parametrize("txt,fmt,basis,dim", [
    ("RGBA", DataFormat.RGBA, -1, None), ("", DataFormat.RGBA, -1, None),
    ("SH1", DataFormat.SH, 1, 4), ("SH4", DataFormat.SH, 4, 13), ("SH9", DataFormat.SH, 9, 28),
    ("SH16", DataFormat.SH, 16, 49), ("SH25", DataFormat.SH, 25, 76),
    ("SG5", DataFormat.SG, 5, 16), ("ASG7", DataFormat.ASG, 7, 22),
    ("RGBA4", DataFormat.RGBA, 4, 13), ("XYZ3", DataFormat.RGBA, 3, 10)])
def test_data_format_parse(txt, fmt, basis, dim):
    d = DataFormat(txt)
    assert (d.format, d.basis_dim, d.data_dim) == (fmt, basis, dim)


def test_data_format_rejects():
    # the number after "SH" is the basis size: it must be a square <= 25
    for bad in ("SH2", "SH3", "SH36", "SH0"):
        with pytest.raises(AssertionError):
            DataFormat(bad)
    with pytest.raises(ValueError):
        DataFormat("S4H")


def test_data_format_repr_roundtrip():
    for txt in ("RGBA", "SH9", "SG5", "ASG7"):
        assert repr(DataFormat(txt)) == txt
        assert DataFormat(repr(DataFormat(txt))) == DataFormat(txt)


def test_tree_data_dim_from_format():
    assert svox.N3Tree(data_format="SH9").data_dim == 28
    assert svox.N3Tree().data_dim == 4
    with pytest.raises(AssertionError):
        svox.N3Tree(data_format="SH9", data_dim=13)


def _renderer(**kw):
    return svox.VolumeRenderer(svox.N3Tree(data_format="SH9"), **kw)


def test_options_defaults():
    o = _renderer()._get_options()
    assert o.step_size == 1e-3 and o.background_brightness == 1.0
    assert (o.format, o.basis_dim, o.min_comp, o.max_comp) == (DataFormat.SH, 9, 0, 8)
    assert o.ndc_width == -1
    assert o.sigma_thresh == 0.0 and o.stop_thresh == 0.0
    assert not o.density_softplus and o.rgb_padding == 0.0


def test_options_fast_and_overrides():
    r = _renderer()
    o = r._get_options(fast=True)
    assert o.sigma_thresh == 1e-2 and o.stop_thresh == 1e-2
    r.stop_thresh = 0.5          # attribute override wins over `fast`
    o = r._get_options(fast=True)
    assert o.sigma_thresh == 1e-2 and o.stop_thresh == 0.5
    r.sigma_thresh = 0.25
    o = r._get_options(fast=False)
    assert o.sigma_thresh == 0.25 and o.stop_thresh == 0.5


def test_options_comp_and_ndc():
    o = _renderer(min_comp=1, max_comp=3)._get_options()
    assert (o.min_comp, o.max_comp) == (1, 3)
    o = _renderer(max_comp=-2)._get_options()
    assert o.max_comp == 7
    o = _renderer(ndc=svox.NDCConfig(width=64, height=48, focal=60.0))._get_options()
    assert (o.ndc_width, o.ndc_height, o.ndc_focal) == (64, 48, 60.0)


def test_options_struct_layout_matches_header():
    # 13 four-byte fields, in the order of the reference's RenderOptions
    from svox_b200.csrc import _COptions
    import ctypes
    assert ctypes.sizeof(_COptions) == 52
    assert [f[0] for f in _COptions._fields_] == [
        "step_size", "background_brightness", "format", "basis_dim", "ndc_width", "ndc_height",
        "ndc_focal", "min_comp", "max_comp", "sigma_thresh", "stop_thresh", "density_softplus",
        "rgb_padding"]


def test_no_cpu_path():
    tree = svox.N3Tree(data_format="SH1")
    with pytest.raises(RuntimeError, match="no CPU"):
        tree(torch.rand(4, 3))
    r = svox.VolumeRenderer(tree)
    d = torch.tensor([[0.0, 0.0, 1.0]])
    with pytest.raises(RuntimeError, match="no CPU"):
        r(svox.Rays(torch.zeros(1, 3), d, d))
    with pytest.raises(RuntimeError, match="no CPU"):
        r.render_persp(torch.eye(4)[:3], width=4, height=4)


def test_spec_validation_rejects_cpu_tensors():
    from svox_b200 import csrc
    tree = svox.N3Tree(data_format="SH1")
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        csrc.query_vertical(tree._spec(), torch.rand(4, 3))


def test_host_side_sh_basis_matches_the_oracle():
    # svox_b200.sh (the counterpart of svox/sh.py) against the oracle's restatement of the
    # kernel-side basis (svox/csrc/rt_kernel.cu:141-181): same polynomials, same order, float
    # round-off apart (the oracle follows the device code's fused multiply-adds).
    import ctypes as C
    import numpy as np
    import torch
    from oracle import oracle as orc
    from svox_b200 import sh
    gen = torch.Generator().manual_seed(7)
    dirs = torch.randn(257, 3, generator=gen)
    dirs = dirs / dirs.norm(dim=-1, keepdim=True)
    lib = orc.lib()
    for deg in range(5):
        n = (deg + 1) ** 2
        mine = sh.eval_sh_bases(deg, dirs).numpy()
        assert mine.shape == (257, n)
        want = np.empty((257, n), np.float32)
        for i in range(257):
            d = np.ascontiguousarray(dirs[i].numpy(), dtype=np.float32)
            lib.orc_sh_basis(C.c_int(n), d.ctypes.data_as(C.c_void_p),
                             want[i].ctypes.data_as(C.c_void_p))
        assert np.abs(mine - want).max() <= 2e-6
        coef = torch.randn(257, 3, n, generator=gen)
        assert torch.allclose(sh.eval_sh(deg, coef, dirs),
                              (coef * torch.from_numpy(mine)[:, None, :]).sum(-1))
