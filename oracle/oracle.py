"""ctypes front end of the C oracle (test infrastructure only).

All arrays are numpy; float32 for coordinates and tree data, int32 for the
child links, float64 for gradients.  See ``svox_oracle.c`` for what each
function restates.
"""
import ctypes as C
import numpy as np

from .build import build_oracle

FORMAT_RGBA, FORMAT_SH, FORMAT_SG, FORMAT_ASG = 0, 1, 2, 3


class OrcTree(C.Structure):
    _fields_ = [("data", C.c_void_p), ("child", C.c_void_p), ("M", C.c_int64),
                ("N", C.c_int32), ("K", C.c_int32),
                ("offset", C.c_float * 3), ("scaling", C.c_float * 3),
                ("extra", C.c_void_p), ("extra_cols", C.c_int32)]


class OrcOptions(C.Structure):
    _fields_ = [("step_size", C.c_float), ("background_brightness", C.c_float),
                ("format", C.c_int32), ("basis_dim", C.c_int32),
                ("ndc_width", C.c_int32), ("ndc_height", C.c_int32),
                ("ndc_focal", C.c_float), ("min_comp", C.c_int32),
                ("max_comp", C.c_int32), ("sigma_thresh", C.c_float),
                ("stop_thresh", C.c_float), ("density_softplus", C.c_int32),
                ("rgb_padding", C.c_float)]


CONTRACT_FIELDS = ["transform", "norm", "pos", "dda_root", "dda_leaf", "sh_dot",
                   "color_pad", "out_acc", "bg_acc", "cam_xy", "cam_rot",
                   "ndc_shift", "sh_basis", "ndc_norm", "descend"]


class OrcContract(C.Structure):
    _fields_ = [(n, C.c_int32) for n in CONTRACT_FIELDS]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_oracle())
        _lib.orc_trace_log.restype = C.c_int64
    return _lib


def get_contract(backward=False):
    """Fused-multiply-add pattern of the forward (or backward) kernels."""
    c = OrcContract()
    lib().orc_get_contract(C.c_int(int(backward)), C.byref(c))
    return {n: getattr(c, n) for n in CONTRACT_FIELDS}


def set_contract(backward=False, **kw):
    cur = get_contract(backward)
    cur.update(kw)
    c = OrcContract(*[cur[n] for n in CONTRACT_FIELDS])
    lib().orc_set_contract(C.c_int(int(backward)), C.byref(c))
    return cur


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    lib().orc_set_num_threads(int(n))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Tree:
    """Borrowed view of the tree arrays: data (M,N,N,N,K) f32, child (M,N,N,N) i32."""

    def __init__(self, data, child, offset=(0, 0, 0), scaling=(1, 1, 1), extra=None):
        self.data = _f32(data)
        self.child = np.ascontiguousarray(child, dtype=np.int32)
        assert self.data.ndim == 5 and self.child.ndim == 4
        self.M, self.N = self.child.shape[0], self.child.shape[1]
        self.K = self.data.shape[-1]
        self.offset = [float(x) for x in np.asarray(offset, dtype=np.float32)]
        self.scaling = [float(x) for x in np.asarray(scaling, dtype=np.float32)]
        # lobe parameters of the SG / ASG colour bases, (basis_dim, 4 or 11)
        self.extra = _f32(extra) if extra is not None and np.size(extra) else None
        self.c = OrcTree(_ptr(self.data), _ptr(self.child), self.M, self.N, self.K,
                         (C.c_float * 3)(*self.offset), (C.c_float * 3)(*self.scaling),
                         _ptr(self.extra), self.extra.shape[1] if self.extra is not None else 0)

    @classmethod
    def from_n3tree(cls, tree, world=True):
        """From any object with svox's N3Tree tensors (data, child, offset, invradius)."""
        n = tree.n_internal if hasattr(tree, "n_internal") else tree.child.shape[0]
        del n  # the kernels see the full capacity, as the reference's do
        data = tree.data.detach().cpu().numpy()
        child = tree.child.cpu().numpy()
        extra = getattr(tree, "extra_data", None)
        extra = extra.cpu().numpy() if extra is not None else None
        if world:
            return cls(data, child, tree.offset.cpu().numpy(), tree.invradius.cpu().numpy(),
                       extra=extra)
        return cls(data, child, extra=extra)


def options(step_size=1e-3, background_brightness=1.0, format=FORMAT_SH, basis_dim=1,
            ndc_width=-1, ndc_height=-1, ndc_focal=0.0, min_comp=0, max_comp=None,
            sigma_thresh=0.0, stop_thresh=0.0, density_softplus=False, rgb_padding=0.0):
    if max_comp is None:
        max_comp = basis_dim - 1
    return OrcOptions(step_size, background_brightness, format, basis_dim, ndc_width,
                      ndc_height, ndc_focal, min_comp, max_comp, sigma_thresh, stop_thresh,
                      int(bool(density_softplus)), rgb_padding)


def out_dim(tree, opt):
    return (tree.K - 1) // opt.basis_dim if opt.format != FORMAT_RGBA else tree.K - 1


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"oracle {what}: corrupt tree (descent left the node array)")


def query_vertical(tree, points):
    pts = _f32(points)
    Q = pts.shape[0]
    vals = np.empty((Q, tree.K), np.float32)
    ids = np.empty((Q,), np.int64)
    _check(lib().orc_query_vertical(C.byref(tree.c), _ptr(pts), C.c_int64(Q), _ptr(vals),
                                    _ptr(ids)), "query_vertical")
    return vals, ids


def assign_vertical(tree, points, values):
    """assign_single_kernel (svox/csrc/svox_kernel.cu:80-89): a copy of ``tree.data`` in which
    the first Kv floats of the leaf of each point hold its row of ``values``; of several
    points in one leaf the LAST one wins here (the reference leaves the winner open)."""
    _, ids = query_vertical(tree, points)
    v = _f32(values)
    data = tree.data.copy().reshape(-1, tree.K)
    data[ids, :v.shape[1]] = v        # numpy keeps the last of repeated indices
    return data.reshape(tree.data.shape)


def calc_corners(parent_depth, N, indexer):
    """calc_corner_kernel (svox/csrc/svox_kernel.cu:91-115): per level, add the cell's
    coordinates then divide by N, in float32, walking parent_depth[:, 0] (the packed index
    of the parent cell) up to the root."""
    pd = np.asarray(parent_depth)
    idx = np.asarray(indexer, dtype=np.int64)
    out = np.zeros((idx.shape[0], 3), np.float32)
    fn = np.float32(N)
    for q in range(idx.shape[0]):
        node, c = int(idx[q, 0]), [int(x) for x in idx[q, 1:]]
        r = np.zeros(3, np.float32)
        while True:
            r = (r + np.asarray(c, np.float32)) / fn
            if node == 0:
                break
            packed = int(pd[node, 0])
            c = [0, 0, 0]
            for a in (2, 1, 0):
                c[a] = packed % N
                packed //= N
            node = packed
        out[q] = r
    return out


def query_vertical_backward(tree, points, grad_out):
    pts = _f32(points)
    g = _f32(grad_out)
    Q, Kg = g.shape
    grad = np.zeros((tree.M, tree.N, tree.N, tree.N, Kg), np.float64)
    _check(lib().orc_query_vertical_backward(C.byref(tree.c), _ptr(pts), C.c_int64(Q), _ptr(g),
                                             C.c_int32(Kg), _ptr(grad)),
           "query_vertical_backward")
    return grad


def volume_render(tree, origins, dirs, vdirs, opt, want_counts=False):
    o, d, v = _f32(origins), _f32(dirs), _f32(vdirs)
    Q = o.shape[0]
    out = np.zeros((Q, out_dim(tree, opt)), np.float32)
    vis = np.zeros(Q, np.int32) if want_counts else None
    con = np.zeros(Q, np.int32) if want_counts else None
    _check(lib().orc_volume_render(C.byref(tree.c), _ptr(o), _ptr(d), _ptr(v), C.c_int64(Q),
                                   C.byref(opt), _ptr(out), _ptr(vis), _ptr(con)),
           "volume_render")
    return (out, vis, con) if want_counts else out


class weight_accumulation:
    """``with weight_accumulation(tree, "sum") as acc:`` -- forward renders inside the block
    accumulate every contributing sample's weight per leaf into ``acc`` (float64, shape of
    ``child``), as the reference does with ``tree.accumulate_weights``
    (svox/svox.py:810-832, svox/csrc/rt_kernel.cu:298-304)."""

    def __init__(self, tree, op="sum"):
        assert op in ("sum", "max")
        self.buf = np.zeros(tree.child.shape, np.float64)
        self.op = op

    def __enter__(self):
        lib().orc_set_weight_accum(_ptr(self.buf), C.c_int(1 if self.op == "max" else 0))
        return self.buf

    def __exit__(self, *exc):
        lib().orc_set_weight_accum(None, C.c_int(0))


def trace_log(tree, origin, dir, vdir, opt, cap=4096):
    o, d, v = _f32(origin), _f32(dir), _f32(vdir)
    slots = np.zeros(cap, np.int64)
    dts = np.zeros(cap, np.float32)
    ts = np.zeros(cap, np.float32)
    out = np.zeros(64, np.float32)
    n = lib().orc_trace_log(C.byref(tree.c), _ptr(o), _ptr(d), _ptr(v), C.byref(opt),
                            C.c_int32(cap), _ptr(slots), _ptr(dts), _ptr(ts), _ptr(out))
    n = min(int(n), cap)
    return slots[:n], dts[:n], ts[:n], out[:out_dim(tree, opt)]


def _grad_buffers(shape, want_abs):
    """grad (and, behind it in the same allocation, the sum of |contributions|)."""
    n = int(np.prod(shape))
    buf = np.zeros(2 * n if want_abs else n, np.float64)
    grad = buf[:n].reshape(shape)
    gabs = buf[n:].reshape(shape) if want_abs else None
    lib().orc_set_grad_abs(_ptr(grad), _ptr(gabs))
    return grad, gabs


def volume_render_backward(tree, origins, dirs, vdirs, opt, grad_out, want_counts=False,
                           want_abs=False):
    """Gradient w.r.t. data (float64).  ``want_abs`` also returns the per-element sum of
    |contributions| (the scale of a float-atomics sum's rounding error)."""
    o, d, v, g = _f32(origins), _f32(dirs), _f32(vdirs), _f32(grad_out)
    Q = o.shape[0]
    grad, gabs = _grad_buffers(tree.data.shape, want_abs)
    vis = np.zeros(Q, np.int32) if want_counts else None
    con = np.zeros(Q, np.int32) if want_counts else None
    _check(lib().orc_volume_render_backward(C.byref(tree.c), _ptr(o), _ptr(d), _ptr(v),
                                            C.c_int64(Q), C.byref(opt), _ptr(g), _ptr(grad),
                                            _ptr(vis), _ptr(con)), "volume_render_backward")
    lib().orc_set_grad_abs(None, None)
    if want_abs:
        return (grad, gabs, vis, con) if want_counts else (grad, gabs)
    return (grad, vis, con) if want_counts else grad


def se_grad(tree, origins, dirs, vdirs, opt, colors, want_abs=False):
    """Rendered colour (float32), gradient and Gauss-Newton diagonal (float64) of
    1/2 sum (render - colors)^2 -- the reference's ``se_grad`` (svox/renderer.py:324-349).
    ``want_abs`` also returns the per-element sum of |gradient contributions|."""
    o, d, v, c = _f32(origins), _f32(dirs), _f32(vdirs), _f32(colors)
    Q = o.shape[0]
    out = np.zeros((Q, out_dim(tree, opt)), np.float32)
    grad, gabs = _grad_buffers(tree.data.shape, want_abs)
    hess = np.zeros(tree.data.shape, np.float64)
    _check(lib().orc_se_grad(C.byref(tree.c), _ptr(o), _ptr(d), _ptr(v), C.c_int64(Q),
                             C.byref(opt), _ptr(c), _ptr(out), _ptr(grad), _ptr(hess)), "se_grad")
    lib().orc_set_grad_abs(None, None)
    return (out, grad, hess, gabs) if want_abs else (out, grad, hess)


def _c2w34(c2w):
    c = _f32(np.asarray(c2w)[:3, :4])
    assert c.shape == (3, 4)
    return c


def volume_render_image(tree, c2w, fx, fy, width, height, opt, want_counts=False):
    c = _c2w34(c2w)
    out = np.zeros((height, width, out_dim(tree, opt)), np.float32)
    Q = width * height
    vis = np.zeros(Q, np.int32) if want_counts else None
    con = np.zeros(Q, np.int32) if want_counts else None
    _check(lib().orc_volume_render_image(C.byref(tree.c), _ptr(c), C.c_float(fx), C.c_float(fy),
                                         C.c_int32(width), C.c_int32(height), C.byref(opt),
                                         _ptr(out), _ptr(vis), _ptr(con)), "volume_render_image")
    return (out, vis, con) if want_counts else out


def volume_render_image_backward(tree, c2w, fx, fy, width, height, opt, grad_out,
                                 want_abs=False):
    c = _c2w34(c2w)
    g = _f32(grad_out)
    grad, gabs = _grad_buffers(tree.data.shape, want_abs)
    _check(lib().orc_volume_render_image_backward(
        C.byref(tree.c), _ptr(c), C.c_float(fx), C.c_float(fy), C.c_int32(width),
        C.c_int32(height), C.byref(opt), _ptr(g), _ptr(grad)), "volume_render_image_backward")
    lib().orc_set_grad_abs(None, None)
    return (grad, gabs) if want_abs else grad


def pixel_rays(c2w, fx, fy, width, height):
    c = _c2w34(c2w)
    o = np.zeros((width * height, 3), np.float32)
    d = np.zeros((width * height, 3), np.float32)
    lib().orc_pixel_rays(_ptr(c), C.c_float(fx), C.c_float(fy), C.c_int32(width),
                         C.c_int32(height), _ptr(o), _ptr(d))
    return o, d
