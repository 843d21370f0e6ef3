"""The C-ABI library: loads, exports every symbol the header declares, and
rejects bad arguments with status codes before touching the GPU (no GPU)."""
import ctypes as C
import os
import re

import pytest

from svox_b200 import csrc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")
HEADER = os.path.join(INCLUDE, "svox_b200.h")


def _strip_comments(text):
    return re.sub(r"/\*.*?\*/", "", text, flags=re.S)


def _declared():
    names = set()
    for fn in sorted(os.listdir(INCLUDE)):
        if fn.endswith(".h"):
            text = _strip_comments(open(os.path.join(INCLUDE, fn)).read())
            names |= set(re.findall(r"\b(svoxb_[a-z_0-9]+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def lib():
    if not csrc.is_built():
        from svox_b200.csrc.build import build
        build()
    return csrc.library()


def test_header_symbols_exported(lib):
    names = _declared()
    assert {"svoxb_query_vertical", "svoxb_query_vertical_backward", "svoxb_volume_render",
            "svoxb_volume_render_image", "svoxb_volume_render_backward",
            "svoxb_volume_render_image_backward", "svoxb_device_status",
            "svoxb_strerror"} <= set(names)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in svox_b200.h but not exported"


def test_strerror_and_version(lib):
    assert lib.svoxb_strerror(0) == b"ok"
    assert b"null" in lib.svoxb_strerror(1)
    assert lib.svoxb_strerror(12345) == b"unknown status"
    assert re.fullmatch(rb"\d+\.\d+\.\d+", lib.svoxb_version())


def test_argument_errors_without_gpu(lib):
    tree = csrc._CTree(0, 0, 0, 0, 1, 2, 4)
    assert lib.svoxb_query_vertical(C.byref(tree), None, C.c_int64(4), None, None, None) == 1
    assert lib.svoxb_query_vertical(None, None, C.c_int64(0), None, None, None) == 1
    ok = csrc._CTree(16, 16, 16, 16, 1, 2, 4)       # non-null dummies, never dereferenced
    assert lib.svoxb_query_vertical(C.byref(ok), None, C.c_int64(-1), None, None, None) == 2
    assert lib.svoxb_query_vertical(C.byref(ok), None, C.c_int64(0), None, None, None) == 0
    bad_n = csrc._CTree(16, 16, 16, 16, 1, 1, 4)
    assert lib.svoxb_query_vertical(C.byref(bad_n), None, C.c_int64(0), None, None, None) == 2
    rays = csrc._CRays(0, 0, 0, 0)
    opt = csrc.RenderOptions()
    opt.format, opt.basis_dim, opt.max_comp = csrc.FORMAT_SG, 1, 0
    o = opt._pack()
    # a Gaussian basis without its lobe parameters, with too few of them, with too many lobes
    assert lib.svoxb_volume_render(C.byref(ok), C.byref(rays), C.byref(o), None, None) == 1
    lobes = csrc._CTree(16, 16, 16, 16, 1, 2, 4, 0, 0, 0, 16, 1, 3)
    assert lib.svoxb_volume_render(C.byref(lobes), C.byref(rays), C.byref(o), None, None) == 2
    lobes = csrc._CTree(16, 16, 16, 16, 1, 2, 4, 0, 0, 0, 16, 1, 4)
    assert lib.svoxb_volume_render(C.byref(lobes), C.byref(rays), C.byref(o), None, None) == 0
    opt.format = csrc.FORMAT_ASG
    o = opt._pack()
    assert lib.svoxb_volume_render(C.byref(lobes), C.byref(rays), C.byref(o), None, None) == 2
    opt.format, opt.basis_dim, opt.max_comp = csrc.FORMAT_SG, 26, 25
    o = opt._pack()
    assert lib.svoxb_volume_render(C.byref(lobes), C.byref(rays), C.byref(o), None, None) == 3
    opt.format = 7
    o = opt._pack()
    assert lib.svoxb_volume_render(C.byref(lobes), C.byref(rays), C.byref(o), None, None) == 3
    # the no-allocation entry point is for SH colour only: a lobe basis is refused before
    # anything is launched
    opt.format, opt.basis_dim, opt.max_comp = csrc.FORMAT_SG, 1, 0
    o = opt._pack()
    assert lib.svoxb_volume_render_noalloc(C.byref(lobes), C.byref(rays), C.byref(o), None,
                                           None) == 3
    opt.format, opt.basis_dim, opt.max_comp = csrc.FORMAT_SH, 2, 1   # not a square
    o = opt._pack()
    assert lib.svoxb_volume_render(C.byref(ok), C.byref(rays), C.byref(o), None, None) == 3
    opt.basis_dim, opt.max_comp, opt.step_size = 1, 0, -1.0
    o = opt._pack()
    assert lib.svoxb_volume_render(C.byref(ok), C.byref(rays), C.byref(o), None, None) == 4
    opt.step_size = 1e-3
    o = opt._pack()
    # empty batch: nothing to do, no launch
    assert lib.svoxb_volume_render(C.byref(ok), C.byref(rays), C.byref(o), None, None) == 0
    assert lib.svoxb_test_knob(99, 0) == 4
