"""Differentiable voxel-marching volume renderer with SH colour.

Drop-in for the reference's ``svox.VolumeRenderer`` on CUDA trees
(svox/renderer.py:57-89 autograd functions, :114-187 constructor, :189-288
``forward``, :290-322 ``render_persp``, :387-426 ``persp_rays``, :432-469
option packing).  Rendering runs in the native library's kernels; there is
no CPU render path in this package.
"""
from collections import namedtuple
from warnings import warn

import torch
from torch import autograd, nn

from . import csrc as _C
from .formats import DataFormat

__all__ = ["VolumeRenderer", "NDCConfig", "Rays", "_VolumeRenderFunction",
           "_VolumeRenderImageFunction"]

# When the tree's data requires grad, the forward records its contributing
# samples so that the backward replays them instead of marching again (costs
# memory: about 40 bytes per contributing sample until the backward has run).
USE_ITEM_LOG = True
# Tests: make the backward ignore what the forward kept and march twice like the reference.
FORCE_TWO_MARCHES = False

# Set by ``svox_b200.distributed.overlap_grad_allreduce``: (n_parts, on_part, on_done,
# reserve_sms).  The replay backward then produces the gradient in n_parts consecutive
# leaf ranges and hands each finished range to on_part (which starts its all-reduce).
GRAD_PARTS = None


# Where the training step's gradient is accumulated: None = a fresh tensor per step; else a
# callable ``like -> tensor`` of that shape (svox_b200.distributed.MulticastGradient hands out
# views of its symmetric-memory buffer, so that the gradient can be summed across GPUs where
# it lies).
GRAD_BUFFER = None


def _zeroed_beside(like):
    """A zero tensor shaped like ``like`` whose fill runs on a side stream; -> (tensor, event
    after which it is zero)."""
    buf = GRAD_BUFFER(like) if GRAD_BUFFER is not None else \
        torch.empty_like(like, memory_format=torch.contiguous_format)
    return buf, _C.zero_beside(buf)


def _claim(ctx):
    """The gradient buffer cleared during the forward, once the current stream may use it."""
    if ctx.grad_buffer is None:
        return None
    buf, done = ctx.grad_buffer
    ctx.grad_buffer = None
    torch.cuda.current_stream(buf.device).wait_event(done)
    return buf


def _replay(tree, src, opt, grad_out, fwd, log, image, zeroed=None):
    """Replay backward, in parts when a gradient hook is installed."""
    if GRAD_PARTS is not None:
        n_parts, on_part, on_done, reserve = GRAD_PARTS
        grad = _C.volume_render_backward_replay_parts(tree, src, opt, grad_out, fwd, log, n_parts,
                                                      on_part, reserve_sms=reserve, image=image,
                                                      zeroed=zeroed)
        on_done()
        return grad
    return _C.volume_render_backward_replay(tree, src, opt, grad_out, fwd, log, image=image,
                                            zeroed=zeroed)

NDCConfig = namedtuple("NDCConfig", ["width", "height", "focal"])
Rays = namedtuple("Rays", ["origins", "dirs", "viewdirs"])


def _rays_spec_from_rays(rays):
    spec = _C.RaysSpec()
    spec.origins = rays.origins
    spec.dirs = rays.dirs
    spec.vdirs = rays.viewdirs
    return spec


def _make_camera_spec(c2w, width, height, fx, fy):
    spec = _C.CameraSpec()
    spec.c2w = c2w
    spec.width = width
    spec.height = height
    spec.fx = fx
    spec.fy = fy
    return spec


def _single_march_ok(opt):
    # The backward pass differentiates the render without thresholds
    # (svox/csrc/rt_kernel.cu:377,441); the saved forward output equals that
    # render only when both thresholds are off.
    return opt.sigma_thresh == 0.0 and opt.stop_thresh == 0.0


def _forward(ctx, data, tree, src, opt, prepared, train, image):
    """Common forward of the two autograd Functions.

    What the backward needs is kept with ``save_for_backward`` (freed with the graph, and an
    in-place edit of the returned render raises instead of silently corrupting the gradient):
    the render itself, whose dot product with the upstream gradient replaces the reference's
    first march, and the item log of a training step.
    """
    ctx.tree, ctx.src, ctx.opt, ctx.image = tree, src, opt, image
    ctx.log_capacity = None
    # `train`: whether a backward can follow (the caller knows the grad mode; in here it
    # is always off, and requires_grad / needs_input_grad ignore torch.no_grad())
    if train is None:
        train = data.requires_grad
    log = None
    ctx.grad_buffer = None
    if train and USE_ITEM_LOG and _C.log_eligible(tree, opt):
        # training step: record the contributing samples for the backward pass, and clear the
        # gradient buffer the backward will add into on a second stream meanwhile (the march
        # leaves a third of the memory bandwidth unused)
        ctx.grad_buffer = _zeroed_beside(tree.data)
        out, (log, ctx.log_capacity) = _C.volume_render_logged(tree, src, opt, image=image)
    elif image:
        out = _C.volume_render_image(tree, src, opt, prepared=prepared)
    else:
        out = _C.volume_render(tree, src, opt, prepared=prepared)
    ctx.data_state = (data._version, tree.data_epoch())
    ctx.keeps_out = train and _single_march_ok(opt)
    if ctx.keeps_out:
        ctx.save_for_backward(*((out,) if log is None else (out, log)))
    return out


def _backward(ctx, grad_out):
    """Common backward: replay of the item log, else one march with the saved render, else
    (``data`` was edited since the forward, or thresholds are on) the reference's two marches,
    which recompute everything from the current ``data`` as the reference does."""
    none = (None,) * 5
    if not ctx.needs_input_grad[0]:
        return (None,) + none
    fwd = log = None
    if ctx.keeps_out and not FORCE_TWO_MARCHES:
        saved = ctx.saved_tensors
        unchanged = ctx.data_state == (ctx.tree.data._version, ctx.tree.data_epoch())
        if unchanged:
            fwd = saved[0]
            if len(saved) > 1:
                log = (saved[1], ctx.log_capacity)
    grad_out = grad_out.contiguous()
    if fwd is not None and log is not None:
        return (_replay(ctx.tree, ctx.src, ctx.opt, grad_out, fwd, log, ctx.image,
                        _claim(ctx)),) + none
    ctx.grad_buffer = None
    if ctx.image:
        return (_C.volume_render_image_backward(ctx.tree, ctx.src, ctx.opt, grad_out, fwd),) + none
    return (_C.volume_render_backward(ctx.tree, ctx.src, ctx.opt, grad_out, fwd),) + none


class _VolumeRenderFunction(autograd.Function):
    """svox/renderer.py:57-72."""

    @staticmethod
    def forward(ctx, data, tree, rays, opt, prepared=None, train=None):
        return _forward(ctx, data, tree, rays, opt, prepared, train, False)

    @staticmethod
    def backward(ctx, grad_out):
        return _backward(ctx, grad_out)


class _VolumeRenderImageFunction(autograd.Function):
    """svox/renderer.py:74-89."""

    @staticmethod
    def forward(ctx, data, tree, cam, opt, prepared=None, train=None):
        return _forward(ctx, data, tree, cam, opt, prepared, train, True)

    @staticmethod
    def backward(ctx, grad_out):
        return _backward(ctx, grad_out)


class _FrozenTree:
    def __init__(self, renderer):
        self.renderer = renderer

    def __enter__(self):
        self.renderer._frozen = {}
        return self.renderer

    def __exit__(self, *exc):
        self.renderer._frozen = None


class VolumeRenderer(nn.Module):
    def __init__(self, tree, step_size: float = 1e-3, background_brightness: float = 1.0,
                 ndc: NDCConfig = None, min_comp: int = 0, max_comp: int = -1,
                 density_softplus: bool = False, rgb_padding: float = 0.0):
        super().__init__()
        self.tree = tree
        self.step_size = step_size
        self.background_brightness = background_brightness
        self.ndc_config = ndc
        self.min_comp = min_comp
        self.max_comp = max_comp
        self.density_softplus = density_softplus
        self.rgb_padding = rgb_padding
        if isinstance(tree.data_format, DataFormat):
            self._data_format = None
        else:
            warn("Legacy N3Tree (pre 0.2.18) without data_format, auto-infering SH deg")
            ddim = tree.data_dim
            self._data_format = DataFormat("") if ddim == 4 else DataFormat(f"SH{(ddim - 1) // 3}")
        self.tree._weight_accum = None
        self._frozen = None     # inside frozen_tree(): {(sigma_thresh, softplus): index tensor}

    def frozen_tree(self):
        """``with renderer.frozen_tree(): ...`` -- a promise that the tree (structure and
        data) is not modified inside the block.  Forward renders in the block then build the
        render index of the tree (annotated child array, leaf table, bricks) once instead of
        on every call, which is what many views of one scene want.  No counterpart in the
        reference; outside the block nothing is kept between calls, because ``tree.data`` can
        be changed through ``.data`` without any version counter noticing."""
        return _FrozenTree(self)

    def _training(self):
        return self.tree.data.requires_grad and torch.is_grad_enabled()

    def _prepared(self, opt):
        if self._frozen is None or self._training():
            return None
        key = (float(opt.sigma_thresh), bool(opt.density_softplus))
        if key not in self._frozen:
            self._frozen[key] = _C.render_scratch(self.tree._spec(), opt)
        return self._frozen[key]

    @property
    def data_format(self):
        return self._data_format or self.tree.data_format

    def _require_cuda(self, cuda):
        if not cuda or not self.tree.data.is_cuda:
            raise RuntimeError(
                "svox_b200 has no CPU render path: move the tree to a CUDA device "
                "(tree.cuda()) and call with cuda=True")

    def forward(self, rays: Rays, cuda=True, fast=False):
        """Render ``(B, 3)`` rays -> ``(B, rgb_dim)``.  Differentiable w.r.t. tree.data."""
        self._require_cuda(cuda)
        opt = self._get_options(fast)
        return _VolumeRenderFunction.apply(self.tree.data, self.tree._spec(),
                                           _rays_spec_from_rays(rays), opt, self._prepared(opt),
                                           self._training())

    def render_persp(self, c2w, width=800, height=800, fx=1111.111, fy=None, cuda=True,
                     fast=False):
        """Render a perspective image -> ``(height, width, rgb_dim)``.  Differentiable."""
        self._require_cuda(cuda)
        if fy is None:
            fy = fx
        c2w = c2w.to(dtype=self.tree.data.dtype, device=self.tree.data.device).contiguous()
        opt = self._get_options(fast)
        return _VolumeRenderImageFunction.apply(
            self.tree.data, self.tree._spec(),
            _make_camera_spec(c2w, width, height, fx, fy), opt, self._prepared(opt),
            self._training())

    def se_grad(self, rays: Rays, colors):
        """Rendered colour, gradient and Gauss-Newton diagonal of the total squared error
        ``1/2 sum_r (C_hat(r) - C(r))^2`` (svox/renderer.py:324-349).

        -> ``colors (B, 3), grad (shape of tree.data), diag_hessian (shape of tree.data)``.
        The diagonal is the squared norm of the Jacobian's columns, as in the reference
        (with ``density_softplus`` plus the reference's own second-order term for the density).
        Octrees with three colour channels of 1, 4, 9, 16 or 25 basis functions (SH, SG or
        ASG) take the route through the item log; every other layout with at most four
        output channels (RGBA, N != 2, other basis sizes) is marched twice (the forward,
        then gradient and diagonal together).
        """
        self._require_cuda(True)
        return self._se_grad(_rays_spec_from_rays(rays), colors, False)

    def se_grad_persp(self, c2w, colors, width=800, height=800, fx=1111.111, fy=None):
        """Image version of :meth:`se_grad` (svox/renderer.py:351-385); ``colors (H, W, 3)``."""
        self._require_cuda(True)
        if fy is None:
            fy = fx
        c2w = c2w.to(dtype=self.tree.data.dtype, device=self.tree.data.device).contiguous()
        return self._se_grad(_make_camera_spec(c2w, width, height, fx, fy), colors, True)

    def _se_grad(self, src, colors, image):
        opt = self._get_options(False)
        # the reference's kernel knows no thresholds (svox/csrc/rt_kernel.cu:537, 590)
        opt.sigma_thresh = opt.stop_thresh = 0.0
        tree = self.tree._spec()
        with torch.no_grad():
            colors = colors.to(device=self.tree.data.device, dtype=self.tree.data.dtype)
            if not _C.log_eligible(tree, opt):
                # any other layout (RGBA, N != 2, other basis sizes): the forward, then one
                # more march for gradient and diagonal
                out = (_C.volume_render_image if image else _C.volume_render)(tree, src, opt)
                grad, hess = _C.se_grad_march(tree, src, opt, out,
                                              colors.reshape(out.shape).contiguous(),
                                              image=image)
                return out, grad, hess
            for _ in range(4):      # a log that was too small is enlarged and the render redone
                out, log = _C.volume_render_logged(tree, src, opt, image=image)
                used = _C.log_chunks_used(log[0])
                _C.log_estimate(wait=True)
                if used > log[1]:
                    continue
                resid = (out - colors.reshape(out.shape)).contiguous()
                grad = _C.volume_render_backward_replay(tree, src, opt, resid, out, log,
                                                        image=image, used=max(used, 1))
                hess = _C.volume_render_hessdiag_replay(tree, src, opt, out, log, max(used, 1),
                                                        image=image)
                return out, grad, hess
        raise RuntimeError("se_grad: the item log kept overflowing")

    @staticmethod
    def persp_rays(c2w, width=800, height=800, fx=1111.111, fy=None):
        """Row-major perspective rays for :meth:`forward` (svox/renderer.py:387-426)."""
        if fy is None:
            fy = fx
        origins = c2w[None, :3, 3].expand(height * width, -1).contiguous()
        yy, xx = torch.meshgrid(torch.arange(height, dtype=torch.float64, device=c2w.device),
                                torch.arange(width, dtype=torch.float64, device=c2w.device),
                                indexing="ij")
        xx = (xx - width * 0.5) / float(fx)
        yy = (yy - height * 0.5) / float(fy)
        dirs = torch.stack((xx, -yy, -torch.ones_like(xx)), dim=-1)
        dirs = (dirs / torch.norm(dirs, dim=-1, keepdim=True)).reshape(-1, 3)
        dirs = torch.matmul(c2w[None, :3, :3].double(), dirs[..., None])[..., 0].float()
        return Rays(origins=origins, dirs=dirs, viewdirs=dirs)

    def _get_options(self, fast=False):
        """RenderOptions with the reference's rules (svox/renderer.py:432-469):
        ``max_comp < 0`` counts from the end, ``fast`` sets both thresholds to
        1e-2, and attributes ``sigma_thresh`` / ``stop_thresh`` set on the
        renderer override either."""
        opts = _C.RenderOptions()
        opts.step_size = self.step_size
        opts.background_brightness = self.background_brightness
        opts.format = self.data_format.format
        opts.basis_dim = self.data_format.basis_dim
        opts.min_comp = self.min_comp
        opts.max_comp = self.max_comp + (opts.basis_dim if self.max_comp < 0 else 0)
        opts.density_softplus = self.density_softplus
        opts.rgb_padding = self.rgb_padding
        if self.ndc_config is not None:
            opts.ndc_width = self.ndc_config.width
            opts.ndc_height = self.ndc_config.height
            opts.ndc_focal = self.ndc_config.focal
        else:
            opts.ndc_width = -1
        opts.sigma_thresh = opts.stop_thresh = 1e-2 if fast else 0.0
        if hasattr(self, "sigma_thresh"):
            opts.sigma_thresh = self.sigma_thresh
        if hasattr(self, "stop_thresh"):
            opts.stop_thresh = self.stop_thresh
        return opts
