"""svoxb_volume_render_noalloc -- the forward render for hosts that must not
allocate device memory (an engine that owns the device heap, an allocation-free
real-time loop, a fixed start-up memory budget).  Its scratch is a static
device array, so this test calls it through the raw C ABI, twice in a row on
different inputs (the array keeps the previous call's contents), and compares
each result with the regular entry point.  Collected last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes as C

import pytest
import torch

from golden.cases import CASES
from svox_b200 import csrc

pytestmark = pytest.mark.gpu
RGB_TOL = 1e-5


def _call(lib, fn, tree, rays, opt, stream):
    ct = csrc._CTree(tree.data.data_ptr(), tree.child.data_ptr(), tree.offset.data_ptr(),
                     tree.invradius.data_ptr(), tree.child.shape[0], tree.N, tree.data_dim)
    o, d, v = rays
    cr = csrc._CRays(o.data_ptr(), d.data_ptr(), v.data_ptr(), o.shape[0])
    co = opt._pack()
    out = torch.full((o.shape[0], 3), float("nan"), device=o.device)
    st = getattr(lib, fn)(C.byref(ct), C.byref(cr), C.byref(co), C.c_void_p(out.data_ptr()),
                          C.c_void_p(stream))
    return st, out


def _cases():
    """Ray cases for each block size the entry point picks: SH4 and SH9 records (640 threads),
    SH16 (512) and SH25 (256)."""
    from svox_b200 import workloads as W
    out = [CASES[n]() for n in ("shell_sh9_rays", "c1_rays", "sh25_rays")]
    sh16 = CASES["query_shell"]()                       # a small SH16 shell tree
    gen = torch.Generator().manual_seed(131)
    with torch.no_grad():
        sh16["tree"].data[..., -1].abs_()               # densities >= 0 as in a scene
    sh16.update(kind="rays", rays=W.sphere_rays(3000, gen, 4.0, 0.2, 0.8))
    return out + [sh16]


def test_noalloc_matches_regular_entry_point_twice(cuda_device):
    import numpy as np
    import parity_util as P
    lib = csrc.library()
    stream = torch.cuda.current_stream().cuda_stream
    for case in _cases():                             # calls in a row on different trees
        tree = case["tree"].to(cuda_device)
        rays = [t.to(cuda_device).contiguous() for t in case["rays"]]
        opt = P.options_of(case)
        st0, want = _call(lib, "svoxb_volume_render", tree, rays, opt, stream)
        st1, got = _call(lib, "svoxb_volume_render_noalloc", tree, rays, opt, stream)
        torch.cuda.synchronize()
        assert st0 == 0 and st1 == 0
        # same kernel, another home for its index: the colours are the same bits
        assert torch.equal(got, want)
        # and again on the same inputs: the left-over scratch does not matter
        st2, again = _call(lib, "svoxb_volume_render_noalloc", tree, rays, opt, stream)
        torch.cuda.synchronize()
        assert st2 == 0 and torch.equal(again, got)
        case["tree"].to("cpu")
        case = dict(case, grad_out=None, mse_targets=None)
        assert np.abs(got.cpu().numpy() - P.run_oracle(case)["out"]).max() <= RGB_TOL
    csrc.check_device_status()


def test_noalloc_refuses_what_it_cannot_hold(cuda_device):
    import svox_b200 as svox
    lib = csrc.library()
    tree = svox.N3Tree(data_format="SH1", init_refine=1).to(cuda_device)
    d = torch.tensor([[0.0, 0.0, 1.0]], device=cuda_device)
    rays = [torch.tensor([[0.1, 0.1, -0.1]], device=cuda_device), d, d]
    opt = svox.VolumeRenderer(tree)._get_options()
    # claim more nodes than the static scratch holds: refused before any launch
    ct = csrc._CTree(tree.data.data_ptr(), tree.child.data_ptr(), tree.offset.data_ptr(),
                     tree.invradius.data_ptr(), (1 << 19) + 1, 2, 4)
    cr = csrc._CRays(rays[0].data_ptr(), rays[1].data_ptr(), rays[2].data_ptr(), 1)
    co = opt._pack()
    out = torch.zeros(1, 3, device=cuda_device)
    st = lib.svoxb_volume_render_noalloc(C.byref(ct), C.byref(cr), C.byref(co),
                                         C.c_void_p(out.data_ptr()), None)
    assert st == 8 and b"maximum" in lib.svoxb_strerror(st)     # SVOXB_ERR_TOO_LARGE
    # RGBA records are not a layout of this variant
    rgba = svox.N3Tree(data_format="RGBA").to(cuda_device)
    ropt = svox.VolumeRenderer(rgba)._get_options()
    ct = csrc._CTree(rgba.data.data_ptr(), rgba.child.data_ptr(), rgba.offset.data_ptr(),
                     rgba.invradius.data_ptr(), 1, 2, 4)
    co = ropt._pack()
    st = lib.svoxb_volume_render_noalloc(C.byref(ct), C.byref(cr), C.byref(co),
                                         C.c_void_p(out.data_ptr()), None)
    assert st == 3                                               # SVOXB_ERR_FORMAT
