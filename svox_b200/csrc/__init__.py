"""Host-side mirror of the reference's native module ``svox.csrc``.

Same spec classes (``TreeSpec``, ``RaysSpec``, ``CameraSpec``,
``RenderOptions``) and the same functions with the same arguments and
results as the reference's pybind11 module (svox/csrc/svox.cpp:63-122), but
implemented by the C-ABI library ``libsvox_b200.so`` (hand-written sm_100a
kernels) loaded with ctypes.  Tensors are allocated by PyTorch and handed to
the library as raw device pointers together with the current CUDA stream.

There is no CPU implementation: if the library is missing or a tensor is
not on a CUDA device, the call raises.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# SVOXB_LIBRARY: load another build of the library (e.g. one compiled with other flags)
LIB_PATH = os.environ.get("SVOXB_LIBRARY") or os.path.join(_HERE, "libsvox_b200.so")

FORMAT_RGBA, FORMAT_SH, FORMAT_SG, FORMAT_ASG = 0, 1, 2, 3
ERR_TOO_LARGE = 8   # svoxb status: a size limit or the scratch allocation


class _CTree(C.Structure):
    _fields_ = [("data", C.c_void_p), ("child", C.c_void_p), ("offset", C.c_void_p),
                ("scaling", C.c_void_p), ("M", C.c_int64), ("N", C.c_int32), ("K", C.c_int32),
                ("weight_accum", C.c_void_p), ("weight_accum_max", C.c_int32),
                ("reserved_", C.c_int32), ("extra_data", C.c_void_p),
                ("extra_rows", C.c_int32), ("extra_cols", C.c_int32)]


class _CRays(C.Structure):
    _fields_ = [("origins", C.c_void_p), ("dirs", C.c_void_p), ("vdirs", C.c_void_p),
                ("Q", C.c_int64)]


class _CCamera(C.Structure):
    _fields_ = [("c2w", C.c_void_p), ("fx", C.c_float), ("fy", C.c_float),
                ("width", C.c_int32), ("height", C.c_int32)]


class _COptions(C.Structure):
    _fields_ = [("step_size", C.c_float), ("background_brightness", C.c_float),
                ("format", C.c_int32), ("basis_dim", C.c_int32), ("ndc_width", C.c_int32),
                ("ndc_height", C.c_int32), ("ndc_focal", C.c_float), ("min_comp", C.c_int32),
                ("max_comp", C.c_int32), ("sigma_thresh", C.c_float),
                ("stop_thresh", C.c_float), ("density_softplus", C.c_int32),
                ("rgb_padding", C.c_float)]


# ---------------------------------------------------------------------------
# Spec objects: plain attribute bags with the reference's field names.

class TreeSpec:
    def __init__(self):
        self.data = self.child = self.parent_depth = self.extra_data = None
        self.offset = self.scaling = None
        self._weight_accum = None
        self._weight_accum_max = False
        self._owner = None          # weak reference to the N3Tree this spec was packed from

    def data_epoch(self):
        """Counter of the owning tree's in-place edits of ``data`` that autograd's version
        counter does not see (``tree[...] = v`` writes through ``data.data``); -1 without
        an owner."""
        tree = self._owner() if self._owner is not None else None
        return tree._data_epoch if tree is not None else -1


class RaysSpec:
    def __init__(self):
        self.origins = self.dirs = self.vdirs = None


class CameraSpec:
    def __init__(self):
        self.c2w = None
        self.fx = self.fy = 0.0
        self.width = self.height = 0


class RenderOptions:
    def __init__(self):
        self.step_size = 1e-3
        self.background_brightness = 1.0
        self.format = FORMAT_RGBA
        self.basis_dim = -1
        self.ndc_width = -1
        self.ndc_height = -1
        self.ndc_focal = 0.0
        self.min_comp = 0
        self.max_comp = 0
        self.sigma_thresh = 0.0
        self.stop_thresh = 0.0
        self.density_softplus = False
        self.rgb_padding = 0.0

    def _pack(self):
        return _COptions(self.step_size, self.background_brightness, int(self.format),
                         int(self.basis_dim), int(self.ndc_width), int(self.ndc_height),
                         float(self.ndc_focal), int(self.min_comp), int(self.max_comp),
                         self.sigma_thresh, self.stop_thresh, int(bool(self.density_softplus)),
                         self.rgb_padding)


# ---------------------------------------------------------------------------
_lib = None


def library():
    """The loaded C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"svox_b200: native library {LIB_PATH} not found; build it with "
                "`python -m svox_b200.csrc.build` (needs nvcc). There is no CPU fallback.")
        lib = C.CDLL(LIB_PATH)
        for name in ("svoxb_strerror", "svoxb_last_cuda_error", "svoxb_version"):
            getattr(lib, name).restype = C.c_char_p
        _lib = lib
    return _lib


def is_built():
    return os.path.exists(LIB_PATH)


def _raise(status, what):
    lib = library()
    msg = lib.svoxb_strerror(int(status)).decode()
    cuda = lib.svoxb_last_cuda_error().decode()
    raise RuntimeError(f"svox_b200.{what}: {msg}" + (f" ({cuda})" if cuda else ""))


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


# Optional per-call device timing (used by the benchmark): when a list is
# installed with ``set_timing``, every library call appends
# (name, start_event, end_event), recorded on the launching stream around the
# call's kernels only (output zero-fill excluded).
_timing = None


def set_timing(records):
    global _timing
    _timing = records


class _timed:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if _timing is not None:
            self.a = torch.cuda.Event(enable_timing=True)
            self.b = torch.cuda.Event(enable_timing=True)
            self.a.record()

    def __exit__(self, *exc):
        if _timing is not None:
            self.b.record()
            _timing.append((self.name, self.a, self.b))


def _check_input(x, name, dtype=torch.float32):
    # mirrors CHECK_INPUT (svox/csrc/include/data_spec.hpp:37-42) plus the dtype
    # check the reference leaves out
    if not torch.is_tensor(x):
        raise RuntimeError(f"{name} must be a tensor")
    if not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not x.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if x.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype} (this build computes in float32 only)")


def _pack_tree(tree):
    for n in ("data", "offset", "scaling"):
        _check_input(getattr(tree, n), n)
    _check_input(tree.child, "child", torch.int32)
    d = tree.data
    if d.dim() != 5 or tree.child.dim() != 4 or tuple(tree.child.shape) != tuple(d.shape[:4]):
        raise RuntimeError("data must be (M,N,N,N,K) and child (M,N,N,N)")
    dev = d.device
    for n in ("child", "offset", "scaling"):
        if getattr(tree, n).device != dev:
            raise RuntimeError(f"{n} must be on the same device as data")
    wa = tree._weight_accum
    wa_ptr = 0
    if wa is not None and wa.numel():
        _check_input(wa, "_weight_accum")
        if tuple(wa.shape) != tuple(tree.child.shape) or wa.device != dev:
            raise RuntimeError("_weight_accum must have the shape and device of child")
        wa_ptr = wa.data_ptr()
    ex = tree.extra_data
    ex_ptr = ex_rows = ex_cols = 0
    if ex is not None and ex.numel():
        _check_input(ex, "extra_data")
        if ex.dim() != 2 or ex.device != dev:
            raise RuntimeError("extra_data must be (basis_dim, C) on the device of data")
        ex_ptr, (ex_rows, ex_cols) = ex.data_ptr(), ex.shape
    return _CTree(d.data_ptr(), tree.child.data_ptr(), tree.offset.data_ptr(),
                  tree.scaling.data_ptr(), d.shape[0], d.shape[1], d.shape[4], wa_ptr,
                  1 if tree._weight_accum_max else 0, 0, ex_ptr, ex_rows, ex_cols)


def _pack_rays(rays, dev):
    for n in ("origins", "dirs", "vdirs"):
        t = getattr(rays, n)
        _check_input(t, n)
        if t.dim() != 2 or t.shape[1] != 3:
            raise RuntimeError(f"{n} must be (Q, 3)")
        if t.device != dev:
            raise RuntimeError(f"{n} must be on the same device as the tree")
    Q = rays.origins.shape[0]
    if rays.dirs.shape[0] != Q or rays.vdirs.shape[0] != Q:
        raise RuntimeError("origins, dirs and vdirs must have the same length")
    return _CRays(rays.origins.data_ptr(), rays.dirs.data_ptr(), rays.vdirs.data_ptr(), Q)


def _pack_camera(cam, dev):
    _check_input(cam.c2w, "c2w")
    if cam.c2w.dim() != 2 or cam.c2w.shape[1] != 4 or cam.c2w.shape[0] not in (3, 4):
        raise RuntimeError("c2w must be (3, 4) or (4, 4)")
    if cam.c2w.device != dev:
        raise RuntimeError("c2w must be on the same device as the tree")
    return _CCamera(cam.c2w.data_ptr(), float(cam.fx), float(cam.fy), int(cam.width),
                    int(cam.height))


def _out_dim(opt, K):
    # get_out_data_dim, svox/csrc/rt_kernel.cu:1009-1015
    return (K - 1) // opt.basis_dim if opt.format != FORMAT_RGBA else K - 1


def _check_indices(indices):
    _check_input(indices, "indices")
    if indices.dim() != 2 or indices.shape[1] != 3:
        raise RuntimeError("indices must be (Q, 3)")


# ---------------------------------------------------------------------------
# Functions of the reference module

def query_vertical(tree, indices):
    """-> (values (Q, K) float32, node_ids (Q,) int64); svox_kernel.cu:120-143."""
    lib = library()
    ct = _pack_tree(tree)
    _check_indices(indices)
    with torch.cuda.device(indices.device):
        Q = indices.shape[0]
        values = torch.empty((Q, ct.K), dtype=indices.dtype, device=indices.device)
        node_ids = torch.empty((Q,), dtype=torch.int64, device=tree.child.device)
        st = lib.svoxb_query_vertical(C.byref(ct), C.c_void_p(indices.data_ptr()), C.c_int64(Q),
                                      C.c_void_p(values.data_ptr()),
                                      C.c_void_p(node_ids.data_ptr()), _stream())
    if st:
        _raise(st, "query_vertical")
    return values, node_ids


_side_streams = {}


def zero_beside(buf):
    """Clear ``buf`` on a side stream of its device, after the work already queued on the
    current stream (the memory's previous users); -> the event after which it is zero.  The
    fill then runs beside whatever the current stream does next."""
    dev = buf.device
    side = _side_streams.get(dev)
    if side is None:
        side = _side_streams[dev] = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        buf.zero_()
        done = torch.cuda.Event()
        done.record(side)
    # should the tensor be dropped before anyone waited for the fill: its memory must not be
    # handed out again while the side stream still writes to it
    if buf.untyped_storage().size() and not _is_symmetric(buf):
        buf.record_stream(side)
    return done


def _is_symmetric(buf):
    """Symmetric-memory allocations do not come from the caching allocator."""
    try:
        from ..distributed import MulticastGradient
    except ImportError:         # torch.distributed not built
        return False
    mc = MulticastGradient.active
    return mc is not None and mc.owns(buf)


def query_vertical_backward(tree, indices, grad_output, zeroed=None):
    """-> gradient w.r.t. data, (M, N, N, N, Kg); svox_kernel.cu:160-182.  ``zeroed``: a zero
    tensor of that shape to add the rows into (else one is made and cleared here)."""
    lib = library()
    ct = _pack_tree(tree)
    _check_indices(indices)
    _check_input(grad_output, "grad_output")
    Q = indices.shape[0]
    if grad_output.dim() != 2 or grad_output.shape[0] != Q:
        raise RuntimeError("grad_output must be (Q, K)")
    Kg = grad_output.shape[1]
    with torch.cuda.device(indices.device):
        shape = (ct.M, ct.N, ct.N, ct.N, Kg)
        if zeroed is not None:
            _check_input(zeroed, "zeroed")
            if tuple(zeroed.shape) != shape:
                raise RuntimeError("zeroed must be (M, N, N, N, Kg)")
        grad = zeroed if zeroed is not None else \
            torch.empty(shape, dtype=grad_output.dtype, device=grad_output.device)
        st = lib.svoxb_query_vertical_backward(
            C.byref(ct), C.c_void_p(indices.data_ptr()), C.c_int64(Q),
            C.c_void_p(grad_output.data_ptr()), C.c_int32(Kg), C.c_void_p(grad.data_ptr()),
            C.c_int(0 if zeroed is not None else 1), _stream())
    if st:
        _raise(st, "query_vertical_backward")
    return grad


def assign_vertical(tree, indices, values):
    """Write row q of ``values`` (Q, Kv <= K) into the record of the leaf that holds point q
    (in place, into ``tree.data``); svox_kernel.cu:80-89,145-158."""
    lib = library()
    ct = _pack_tree(tree)
    _check_indices(indices)
    _check_input(values, "values")
    Q = indices.shape[0]
    if values.dim() != 2 or values.shape[0] != Q or not 1 <= values.shape[1] <= ct.K:
        raise RuntimeError("values must be (Q, Kv) with 1 <= Kv <= K")
    with torch.cuda.device(indices.device):
        st = lib.svoxb_assign_vertical(
            C.byref(ct), C.c_void_p(indices.data_ptr()), C.c_int64(Q),
            C.c_void_p(values.data_ptr()), C.c_int32(values.shape[1]),
            C.c_void_p(tree.data.data_ptr()), _stream())
    if st:
        _raise(st, "assign_vertical")


def calc_corners(tree, indexer):
    """Lower corners (Q, 3), tree-local, of the cells ``indexer`` (Q, 4) int64 =
    (node, i, j, k); svox_kernel.cu:91-115,184-203."""
    lib = library()
    ct = _pack_tree(tree)
    _check_input(indexer, "indexer", torch.int64)
    _check_input(tree.parent_depth, "parent_depth", torch.int32)
    if indexer.dim() != 2 or indexer.shape[1] != 4:
        raise RuntimeError("indexer must be (Q, 4)")
    if tuple(tree.parent_depth.shape) != (ct.M, 2) or tree.parent_depth.device != indexer.device:
        raise RuntimeError("parent_depth must be (M, 2) on the device of indexer")
    Q = indexer.shape[0]
    with torch.cuda.device(indexer.device):
        out = torch.empty((Q, 3), dtype=tree.data.dtype, device=indexer.device)
        st = lib.svoxb_calc_corners(
            C.byref(ct), C.c_void_p(tree.parent_depth.data_ptr()),
            C.c_void_p(indexer.data_ptr()), C.c_int64(Q), C.c_void_p(out.data_ptr()),
            _stream())
    if st:
        _raise(st, "calc_corners")
    return out


def render_scratch(tree, opt):
    """The forward render's index of the tree (density-annotated child array, leaf table,
    bricks) as an int32 tensor, for ``volume_render[_image](..., prepared=...)``: valid until
    the tree, ``opt.sigma_thresh`` or ``opt.density_softplus`` change.  None if this tree /
    format renders through kernels that keep no such index."""
    lib = library()
    ct = _pack_tree(tree)
    co = opt._pack()
    lib.svoxb_render_scratch_words.restype = C.c_int64
    words = lib.svoxb_render_scratch_words(C.byref(ct))
    if words <= 0:
        return None
    with torch.cuda.device(tree.data.device):
        scratch = torch.empty(words, dtype=torch.int32, device=tree.data.device)
        st = lib.svoxb_render_scratch_build(C.byref(ct), C.byref(co),
                                            C.c_void_p(scratch.data_ptr()), _stream())
    if st in (3, 4, ERR_TOO_LARGE):      # format / option / size the queue kernels do not take
        return None
    if st:
        _raise(st, "render_scratch_build")
    return scratch


def volume_render(tree, rays, opt, prepared=None):
    """-> (Q, out_dim); svox/csrc/rt_kernel.cu:1019-1036.  ``prepared``: a tensor from
    ``render_scratch`` for the same tree and options (skips the per-call index build)."""
    lib = library()
    ct = _pack_tree(tree)
    cr = _pack_rays(rays, tree.data.device)
    co = opt._pack()
    with torch.cuda.device(tree.data.device):
        out = torch.empty((cr.Q, _out_dim(opt, ct.K)), dtype=torch.float32,
                          device=tree.data.device)
        with _timed("volume_render"):
            if prepared is not None:
                st = lib.svoxb_volume_render_prepared(
                    C.byref(ct), C.byref(cr), C.byref(co), C.c_void_p(prepared.data_ptr()),
                    C.c_void_p(out.data_ptr()), _stream())
            else:
                st = lib.svoxb_volume_render(C.byref(ct), C.byref(cr), C.byref(co),
                                             C.c_void_p(out.data_ptr()), _stream())
    if st:
        _raise(st, "volume_render")
    return out


def volume_render_image(tree, cam, opt, prepared=None):
    """-> (height, width, out_dim); svox/csrc/rt_kernel.cu:1038-1057.  ``prepared`` as for
    ``volume_render``."""
    lib = library()
    ct = _pack_tree(tree)
    cc = _pack_camera(cam, tree.data.device)
    co = opt._pack()
    with torch.cuda.device(tree.data.device):
        out = torch.empty((cc.height, cc.width, _out_dim(opt, ct.K)), dtype=torch.float32,
                          device=tree.data.device)
        if prepared is not None:
            st = lib.svoxb_volume_render_image_prepared(
                C.byref(ct), C.byref(cc), C.byref(co), C.c_void_p(prepared.data_ptr()),
                C.c_void_p(out.data_ptr()), _stream())
        else:
            st = lib.svoxb_volume_render_image(C.byref(ct), C.byref(cc), C.byref(co),
                                               C.c_void_p(out.data_ptr()), _stream())
    if st:
        _raise(st, "volume_render_image")
    return out


# ---------------------------------------------------------------------------
# Logged forward / replay backward (training step without a second march)

# Layout of the log's head (render_queue.cuh): word 0 = chunks the forward asked for,
# word 2 = bin shift, word 3 = number of bins, words LOG_HIST .. LOG_HIST + LOG_MAX_BINS =
# samples per bin of the last logged forward.
LOG_HIST, LOG_MAX_BINS = 32, 1024
_LOG_SLACK_CHUNKS = 2 * 16384   # every warp of the forward takes log chunks 8 at a time
_items_per_ray = 48.0           # running estimate used to size the item log
_WATCH_SLOTS = 8


class _LogWatch:
    """Learns how large the item log has to be WITHOUT making the host wait for the device.

    After a logged forward the number of chunks it asked for is copied to pinned host
    memory, asynchronously; whenever the next log is sized, the counts that have arrived by
    then adapt the per-ray estimate.  A log that was too small costs that one step a marching
    backward (decided on the device, see ``volume_render_backward_replay``), never a wrong
    gradient."""
    slots = {}     # device -> [pinned int32 ring, next slot, pending [(slot, event, rays, cap)]]

    @classmethod
    def _state(cls, device):
        st = cls.slots.get(device)
        if st is None:
            st = [torch.zeros(_WATCH_SLOTS, dtype=torch.int32).pin_memory(), 0, []]
            cls.slots[device] = st
        return st

    @classmethod
    def watch(cls, log, cap, n_rays):
        st = cls._state(log.device)
        pending = st[2]
        if len(pending) >= _WATCH_SLOTS:           # nobody has polled for a while
            cls.poll(log.device, wait=True)
        slot = st[1]
        st[1] = (slot + 1) % _WATCH_SLOTS
        st[0][slot:slot + 1].copy_(log[:1], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        pending.append((slot, ev, n_rays, cap))

    @classmethod
    def poll(cls, device=None, wait=False):
        """Fold the counts that have arrived into the estimate; ``wait`` blocks for all."""
        global _items_per_ray
        for dev, st in cls.slots.items():
            if device is not None and dev != device:
                continue
            keep = []
            for slot, ev, n_rays, cap in st[2]:
                if wait:
                    ev.synchronize()
                elif not ev.query():
                    keep.append((slot, ev, n_rays, cap))
                    continue
                used = int(st[0][slot])
                cls.last_used, cls.last_cap = used, cap
                if n_rays:
                    # chunks are 32 items, partly filled ones included: keep 25 % head room
                    need = max(8.0, 1.25 * 32.0 * used / n_rays)
                    _items_per_ray = need if used > cap else max(need, 0.9 * _items_per_ray)
            st[2] = keep
        return _items_per_ray

    last_used = last_cap = 0


def log_estimate(wait=False):
    """Current estimate of contributing samples per ray (what the next item log is sized by),
    after folding in the counts of finished forwards; ``wait=True`` waits for all of them."""
    return _LogWatch.poll(wait=wait)


def log_eligible(tree, opt):
    """Whether the logged forward / replay backward pair applies to this call."""
    return (opt.format != FORMAT_RGBA and opt.basis_dim in (1, 4, 9, 16, 25)
            and tree.data.shape[1] == 2 and tree.data.shape[4] == 3 * opt.basis_dim + 1
            and opt.sigma_thresh == 0.0 and opt.stop_thresh == 0.0
            and tree.data.dtype == torch.float32)


def _log_alloc(n_rays, device):
    lib = library()
    lib.svoxb_item_log_words.restype = C.c_int64
    _LogWatch.poll(device)
    cap = int(n_rays * _items_per_ray / 32) + _LOG_SLACK_CHUNKS
    words = lib.svoxb_item_log_words(C.c_int64(cap))
    return torch.empty(words, dtype=torch.int32, device=device), cap


def volume_render_logged(tree, rays_or_cam, opt, image=False):
    """Forward render that also records its contributing samples.

    -> (out, (log, capacity_chunks)); pass the pair to ``volume_render_backward_replay``.
    """
    lib = library()
    ct = _pack_tree(tree)
    co = opt._pack()
    dev = tree.data.device
    with torch.cuda.device(dev):
        if image:
            cs = _pack_camera(rays_or_cam, dev)
            shape, n = (cs.height, cs.width, 3), cs.height * cs.width
            fn = lib.svoxb_volume_render_image_logged
        else:
            cs = _pack_rays(rays_or_cam, dev)
            shape, n = (cs.Q, 3), cs.Q
            fn = lib.svoxb_volume_render_logged
        out = torch.empty(shape, dtype=torch.float32, device=dev)
        log, cap = _log_alloc(n, dev)
        with _timed("volume_render"):
            st = fn(C.byref(ct), C.byref(cs), C.byref(co), C.c_void_p(out.data_ptr()),
                    C.c_void_p(log.data_ptr()), C.c_int64(cap), _stream())
        if st:
            _raise(st, "volume_render_logged")
        _LogWatch.watch(log, cap, n)
    return out, (log, cap)


def log_chunks_used(log):
    """Chunks the logged forward asked for (synchronises the current stream)."""
    used = C.c_int64(0)
    st = library().svoxb_item_log_used(C.c_void_p(log.data_ptr()), C.byref(used), _stream())
    if st:
        _raise(st, "item_log_used")
    return used.value


def volume_render_backward_replay(tree, rays_or_cam, opt, grad_output, fwd_out, logpair,
                                  image=False, used=0, zeroed=None):
    """Gradient w.r.t. data from the item log of ``volume_render_logged``.

    ``used=0``: the host does not know whether the log was large enough and does not wait to
    find out -- the kernels check on the device, and a marching backward enqueued behind them
    takes over in that case.  ``used`` > 0: a count read with ``log_chunks_used`` that fits
    the capacity (smaller scratch, no fallback enqueued).  ``zeroed``: a zero tensor like
    ``data`` to add the gradient into (else one is made here)."""
    lib = library()
    log, cap = logpair
    dev = tree.data.device
    with torch.cuda.device(dev):
        ct = _pack_tree(tree)
        co = opt._pack()
        _check_input(grad_output, "grad_output")
        _check_input(fwd_out, "fwd_out")
        if used > cap:
            raise RuntimeError("the item log overflowed: it cannot be replayed")
        grad = zeroed if zeroed is not None else \
            torch.zeros_like(tree.data, memory_format=torch.contiguous_format)
        if image:
            cs = _pack_camera(rays_or_cam, dev)
            fn = lib.svoxb_volume_render_image_backward_replay
        else:
            cs = _pack_rays(rays_or_cam, dev)
            fn = lib.svoxb_volume_render_backward_replay
        with _timed("volume_render_backward"):
            st = fn(C.byref(ct), C.byref(cs), C.byref(co), C.c_void_p(grad_output.data_ptr()),
                    C.c_void_p(fwd_out.data_ptr()), C.c_void_p(log.data_ptr()), C.c_int64(cap),
                    C.c_int64(used), C.c_void_p(grad.data_ptr()), C.c_int(0), _stream())
    if st:
        _raise(st, "volume_render_backward_replay")
    return grad


def volume_render_hessdiag_replay(tree, rays_or_cam, opt, fwd_out, logpair, used, image=False):
    """Gauss-Newton diagonal of the squared error from the item log (third result of the
    reference's ``se_grad``).  ``used``: the count from ``log_chunks_used`` (there is no
    marching fallback for this result, so the caller has to know that the log was large
    enough)."""
    lib = library()
    log, cap = logpair
    dev = tree.data.device
    if not 0 < used <= cap:
        raise RuntimeError("the item log overflowed or its chunk count is not known")
    with torch.cuda.device(dev):
        ct = _pack_tree(tree)
        co = opt._pack()
        _check_input(fwd_out, "fwd_out")
        hess = torch.zeros_like(tree.data, memory_format=torch.contiguous_format)
        if image:
            cs = _pack_camera(rays_or_cam, dev)
            fn = lib.svoxb_volume_render_image_hessdiag_replay
        else:
            cs = _pack_rays(rays_or_cam, dev)
            fn = lib.svoxb_volume_render_hessdiag_replay
        st = fn(C.byref(ct), C.byref(cs), C.byref(co), C.c_void_p(fwd_out.data_ptr()),
                C.c_void_p(log.data_ptr()), C.c_int64(cap), C.c_int64(used),
                C.c_void_p(hess.data_ptr()), C.c_int(0), _stream())
    if st:
        _raise(st, "volume_render_hessdiag_replay")
    return hess


def se_grad_march(tree, rays_or_cam, opt, fwd_out, colors, image=False):
    """-> (grad, hessdiag) of the squared error ``1/2 sum (fwd_out - colors)^2`` by marching
    the rays once more: any record layout with at most four output channels.  ``fwd_out``: the
    render of the same inputs with both thresholds zero."""
    lib = library()
    dev = tree.data.device
    with torch.cuda.device(dev):
        ct = _pack_tree(tree)
        co = opt._pack()
        _check_input(fwd_out, "fwd_out")
        _check_input(colors, "colors")
        if colors.numel() != fwd_out.numel():
            raise RuntimeError("colors must have the shape of the render")
        grad = torch.zeros_like(tree.data, memory_format=torch.contiguous_format)
        hess = torch.zeros_like(grad)
        if image:
            cs = _pack_camera(rays_or_cam, dev)
            fn = lib.svoxb_se_grad_image_march
        else:
            cs = _pack_rays(rays_or_cam, dev)
            fn = lib.svoxb_se_grad_march
        st = fn(C.byref(ct), C.byref(cs), C.byref(co), C.c_void_p(fwd_out.data_ptr()),
                C.c_void_p(colors.data_ptr()), C.c_void_p(grad.data_ptr()),
                C.c_void_p(hess.data_ptr()), C.c_int(0), _stream())
    if st:
        _raise(st, "se_grad_march")
    return grad, hess


def allreduce_multimem(multicast_ptr, n_floats, rank, world):
    """Sum ``n_floats`` floats over the GPUs of a multicast object, in place, on the current
    stream (see ``svoxb_allreduce_multimem``); the caller provides the barriers around it."""
    st = library().svoxb_allreduce_multimem(C.c_void_p(int(multicast_ptr)), C.c_int64(n_floats),
                                            C.c_int(rank), C.c_int(world), _stream())
    if st:
        _raise(st, "allreduce_multimem")


def replay_part_ranges(M, K, n_parts):
    """Leaf-slot ranges [(begin, end)] of the ``n_parts`` parts of a replay backward for a tree
    of ``M`` nodes with ``K`` floats per record (whole bins; the same on every process)."""
    shift = library().svoxb_replay_bin_shift(C.c_int64(M), C.c_int32(K))
    n_slots = M * 8
    n_bins = ((n_slots - 1) >> shift) + 1
    cut = [min(((p * n_bins) // n_parts) << shift, n_slots) for p in range(n_parts)] + [n_slots]
    return list(zip(cut[:-1], cut[1:]))


def volume_render_backward_replay_parts(tree, rays_or_cam, opt, grad_output, fwd_out, logpair,
                                        n_parts, on_part, reserve_sms=0, image=False,
                                        zeroed=None):
    """The replay backward in ``n_parts`` consecutive leaf ranges.  After each part
    ``on_part(rows)`` is called with the flat view of the gradient rows that are final
    (e.g. to start their all-reduce while the next part is computed).  The host never waits
    for the device: whether the log was large enough is decided there, and the marching
    fallback runs before the first part, so the rows handed on are final either way and every
    process of a data-parallel job makes the same ``on_part`` calls."""
    lib = library()
    log, cap = logpair
    dev = tree.data.device
    K = tree.data.shape[-1]
    with torch.cuda.device(dev):
        ct = _pack_tree(tree)
        co = opt._pack()
        _check_input(grad_output, "grad_output")
        _check_input(fwd_out, "fwd_out")
        if image:
            cs = _pack_camera(rays_or_cam, dev)
            begin = lib.svoxb_replay_image_begin
        else:
            cs = _pack_rays(rays_or_cam, dev)
            begin = lib.svoxb_replay_begin
        grad = zeroed if zeroed is not None else \
            torch.zeros_like(tree.data, memory_format=torch.contiguous_format)
        flat = grad.view(-1)
        ranges = replay_part_ranges(ct.M, K, n_parts)
        job = C.c_void_p(None)
        with _timed("volume_render_backward"):
            st = begin(C.byref(ct), C.byref(cs), C.byref(co),
                       C.c_void_p(grad_output.data_ptr()), C.c_void_p(fwd_out.data_ptr()),
                       C.c_void_p(log.data_ptr()), C.c_int64(cap), C.c_int64(0),
                       C.c_int(n_parts), C.c_void_p(grad.data_ptr()), _stream(), C.byref(job))
            if st == ERR_TOO_LARGE:
                # no room for the sorted samples: march; the parts are then final at once
                fn = lib.svoxb_volume_render_image_backward if image \
                    else lib.svoxb_volume_render_backward
                st = fn(C.byref(ct), C.byref(cs), C.byref(co),
                        C.c_void_p(grad_output.data_ptr()), C.c_void_p(fwd_out.data_ptr()),
                        C.c_void_p(grad.data_ptr()), C.c_int(0), _stream())
                if st:
                    _raise(st, "volume_render_backward")
                for lo, hi in ranges:
                    on_part(flat[lo * K:hi * K])
                return grad
            if st:
                _raise(st, "replay_begin")
            try:
                lo, hi = C.c_int64(0), C.c_int64(0)
                for part in range(n_parts):
                    st = lib.svoxb_replay_scatter(job, C.c_int(part), C.c_void_p(grad.data_ptr()),
                                                  C.c_int(reserve_sms), _stream())
                    if st:
                        _raise(st, "replay_scatter")
                    lib.svoxb_replay_part_range(job, C.c_int(part), C.byref(lo), C.byref(hi))
                    assert (lo.value, hi.value) == ranges[part]
                    on_part(flat[lo.value * K:hi.value * K])
            finally:
                lib.svoxb_replay_end(job, _stream())
    return grad


def _fwd_ptr(fwd_out, shape):
    if fwd_out is None:
        return C.c_void_p(0)
    _check_input(fwd_out, "fwd_out")
    if tuple(fwd_out.shape) != tuple(shape):
        raise RuntimeError("fwd_out must have the shape of the forward output")
    return C.c_void_p(fwd_out.data_ptr())


def volume_render_backward(tree, rays, opt, grad_output, fwd_out=None):
    """-> gradient w.r.t. data (like data); svox/csrc/rt_kernel.cu:1059-1083.

    ``fwd_out`` (optional, not in the reference signature) is the forward
    result for the same inputs; it lets the kernel march each ray once.
    """
    lib = library()
    ct = _pack_tree(tree)
    cr = _pack_rays(rays, tree.data.device)
    co = opt._pack()
    _check_input(grad_output, "grad_output")
    shape = (cr.Q, _out_dim(opt, ct.K))
    if tuple(grad_output.shape) != shape:
        raise RuntimeError(f"grad_output must be {shape}")
    with torch.cuda.device(tree.data.device):
        grad = torch.zeros_like(tree.data, memory_format=torch.contiguous_format)
        with _timed("volume_render_backward"):
            st = lib.svoxb_volume_render_backward(
                C.byref(ct), C.byref(cr), C.byref(co), C.c_void_p(grad_output.data_ptr()),
                _fwd_ptr(fwd_out, shape), C.c_void_p(grad.data_ptr()), C.c_int(0), _stream())
    if st:
        _raise(st, "volume_render_backward")
    return grad


def volume_render_image_backward(tree, cam, opt, grad_output, fwd_out=None):
    """-> gradient w.r.t. data; svox/csrc/rt_kernel.cu:1085-1109."""
    lib = library()
    ct = _pack_tree(tree)
    cc = _pack_camera(cam, tree.data.device)
    co = opt._pack()
    _check_input(grad_output, "grad_output")
    shape = (cc.height, cc.width, _out_dim(opt, ct.K))
    if tuple(grad_output.shape) != shape:
        raise RuntimeError(f"grad_output must be {shape}")
    with torch.cuda.device(tree.data.device):
        grad = torch.empty_like(tree.data, memory_format=torch.contiguous_format)
        st = lib.svoxb_volume_render_image_backward(
            C.byref(ct), C.byref(cc), C.byref(co), C.c_void_p(grad_output.data_ptr()),
            _fwd_ptr(fwd_out, shape), C.c_void_p(grad.data_ptr()), C.c_int(1), _stream())
    if st:
        _raise(st, "volume_render_image_backward")
    return grad


def march_stats(tree, rays, opt):
    """Per-ray (visits, contributing samples forward, contributing samples backward),
    three (Q,) int32 tensors (no counterpart in the reference)."""
    lib = library()
    ct = _pack_tree(tree)
    cr = _pack_rays(rays, tree.data.device)
    co = opt._pack()
    with torch.cuda.device(tree.data.device):
        outs = [torch.zeros(cr.Q, dtype=torch.int32, device=tree.data.device) for _ in range(3)]
        st = lib.svoxb_march_stats(C.byref(ct), C.byref(cr), C.byref(co),
                                   *[C.c_void_p(t.data_ptr()) for t in outs], _stream())
    if st:
        _raise(st, "march_stats")
    return tuple(outs)


def device_status(clear=True):
    """Synchronise and return the device anomaly word (0 = none), see svox_b200.h."""
    return int(library().svoxb_device_status(C.c_int(int(clear)), _stream()))


def check_device_status():
    st = device_status(clear=True)
    if st:
        _raise(st, "device_status")


def reserve_sms(n):
    """Leave ``n`` multiprocessors to other kernels (a collective on another stream) in the
    library's persistent kernels; returns the previous setting (``n < 0``: query only)."""
    return int(library().svoxb_reserve_sms(C.c_int(int(n))))


def version():
    return library().svoxb_version().decode()
