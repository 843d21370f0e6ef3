"""The four argument structs of the C ABI have ONE layout: the header's.

A binding that declares a shorter or reordered struct hands the library the
bytes that happen to follow (for ``svoxb_tree`` a wild ``weight_accum``
pointer the forward render would add weights into), so the three places that
spell the layout out are compared field by field: ``include/svox_b200.h``,
the ctypes mirrors in ``svox_b200/csrc`` and the from-scratch binding shown
in ``INTEGRATION.md``.  Reference side: svox/csrc/include/data_spec.hpp:51-126.
"""
import ctypes as C
import os
import re

import pytest

from svox_b200 import csrc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# C type of a header field -> the ctypes type a mirror must use
_CTYPES = {"float": C.c_float, "int32_t": C.c_int32, "int64_t": C.c_int64}
MIRRORS = {"svoxb_tree": csrc._CTree, "svoxb_rays": csrc._CRays, "svoxb_camera": csrc._CCamera,
           "svoxb_render_options": csrc._COptions}
DOC_NAMES = {"svoxb_tree": "Tree", "svoxb_rays": "Rays", "svoxb_camera": "Camera",
             "svoxb_render_options": "Options"}


def header_structs():
    text = open(os.path.join(ROOT, "include", "svox_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for body, name in re.findall(r"typedef\s+struct\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            m = re.fullmatch(r"(const\s+)?(\w+)\s*(\*?)\s*(\w+)", decl)
            assert m, f"cannot parse field {decl!r} of {name}"
            fields.append((m.group(4), C.c_void_p if m.group(3) else _CTYPES[m.group(2)]))
        out[name] = fields
    return out


def doc_structs():
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    out = {}
    for name, body in re.findall(r"class (\w+)\(C\.Structure\):.*?_fields_ = \[(.*?)\]\n", text,
                                 flags=re.S):
        out[name] = [(f, getattr(C, t)) for f, t in re.findall(r'\("(\w+)",\s*C\.(\w+)\)', body)]
    return out


def _layout(fields):
    class S(C.Structure):
        _fields_ = fields
    return [(n, getattr(S, n).offset, getattr(S, n).size) for n, _ in fields], C.sizeof(S)


@pytest.mark.parametrize("name", list(MIRRORS))
def test_ctypes_mirror_matches_header(name):
    want = header_structs()[name]
    mirror = MIRRORS[name]
    got = [(n, t) for n, t in mirror._fields_]
    assert [n for n, _ in got] == [n for n, _ in want]
    assert _layout(got) == _layout(want)
    assert C.sizeof(mirror) == _layout(want)[1]


@pytest.mark.parametrize("name", list(MIRRORS))
def test_integration_document_matches_header(name):
    want = header_structs()[name]
    doc = doc_structs()
    assert DOC_NAMES[name] in doc, f"INTEGRATION.md shows no binding for {name}"
    got = doc[DOC_NAMES[name]]
    assert [n for n, _ in got] == [n for n, _ in want]
    assert _layout(got) == _layout(want)


def test_sizes_are_the_documented_ones():
    h = header_structs()
    assert _layout(h["svoxb_tree"])[1] == 80
    assert _layout(h["svoxb_rays"])[1] == 32
    assert _layout(h["svoxb_camera"])[1] == 24
    assert _layout(h["svoxb_render_options"])[1] == 52     # RenderOptions: 13 x 4 bytes
