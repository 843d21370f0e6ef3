"""Multi-GPU use of the render path: rays are sharded, the tree is replicated.

Rays are independent given a read-only tree, so each rank renders a
contiguous slice of the batch with no communication; the only exchange is one
sum all-reduce of the dense ``tree.data.grad`` after the backward pass.  One
process per GPU (``torchrun``); works with any ``torch.distributed`` backend
(NCCL on GPUs, gloo in the CPU tests).
"""
import torch
import torch.distributed as dist

from .render import Rays

__all__ = ["shard_bounds", "shard_rays", "shard_rows", "allreduce_grad", "broadcast_tree",
           "gather_rows", "overlap_grad_allreduce"]


def _rank_world(rank, world):
    if rank is None or world is None:
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
        return 0, 1
    return rank, world


def shard_bounds(n, rank=None, world=None):
    """[lo, hi) of this rank's contiguous slice of ``n`` items (sizes differ by at most 1)."""
    rank, world = _rank_world(rank, world)
    return rank * n // world, (rank + 1) * n // world


def shard_rows(t, rank=None, world=None):
    lo, hi = shard_bounds(t.shape[0], rank, world)
    return t[lo:hi].contiguous()


def shard_rays(rays, rank=None, world=None):
    """This rank's slice of a ``Rays`` batch."""
    return Rays(*[shard_rows(t, rank, world) for t in rays])


class _Overlap:
    """State of the overlapped gradient all-reduce (see ``overlap_grad_allreduce``)."""
    group = None
    works = []
    reduced = False     # the gradient of the last backward left the renderer already summed

    @classmethod
    def on_part(cls, rows):
        if rows.numel() == 0:       # the same ranges are empty on every rank
            return
        cls.works.append(dist.all_reduce(rows, op=dist.ReduceOp.SUM, group=cls.group,
                                         async_op=True))

    @classmethod
    def agree(cls, ok, log):
        # Every rank must take the same route (the parts run one collective each), and only
        # the leaf ranges that received samples on SOME rank need reducing: sum the ranks'
        # "cannot replay" flags and their per-bin sample counts in one small all-reduce.
        from .csrc import LOG_HIST, LOG_MAX_BINS
        vec = torch.empty(1 + LOG_MAX_BINS, dtype=torch.int64, device=log.device)
        vec[0] = 0 if ok else 1
        vec[1:] = log[LOG_HIST:LOG_HIST + LOG_MAX_BINS]
        dist.all_reduce(vec, op=dist.ReduceOp.SUM, group=cls.group)
        host = vec.cpu()
        n_bins = int(log[3].item())
        if int(host[0]) != 0:
            return False
        used = torch.nonzero(host[1:1 + n_bins]).flatten()
        if used.numel() == 0:
            return (0, 0)
        return (int(used[0]), int(used[-1]) + 1)

    @classmethod
    def on_done(cls):
        for w in cls.works:
            w.wait()            # the current stream waits for the collective's stream
        cls.works = []
        cls.reduced = True


def overlap_grad_allreduce(n_parts=8, group=None, reserve_sms=16):
    """Overlap the all-reduce of ``data.grad`` with its computation, and reduce only the
    leaf ranges that received samples on some rank (the rest of the gradient is zero
    everywhere).  ``n_parts=1`` keeps the second saving without the overlap.

    The replay backward of the renderer produces the gradient leaf range by leaf range;
    with this switched on, the rows of a finished range are all-reduced (asynchronously, on
    the backend's stream) while the next range is computed, and ``reserve_sms`` SMs are left
    to the collective's kernel.  ``allreduce_grad`` then finds the gradient already summed
    and does nothing.  Steps whose backward cannot take that route on some rank (log overflow, options
    the replay does not cover) still get the plain all-reduce; the ranks agree on the route
    with a one-word all-reduce per step.  ``n_parts=0`` switches it off.
    Every rank must make the same call.
    """
    from . import render
    if not n_parts or not (dist.is_available() and dist.is_initialized()) \
            or dist.get_world_size(group) == 1:
        render.GRAD_PARTS = None
        return
    _Overlap.group = group
    _Overlap.works = []
    _Overlap.reduced = False
    render.GRAD_PARTS = (int(n_parts), _Overlap.on_part, _Overlap.on_done, _Overlap.agree,
                         int(reserve_sms) if n_parts > 1 else 0)   # one part: nothing overlaps


def allreduce_grad(tree, group=None, async_op=False):
    """Sum ``tree.data.grad`` over all ranks (the one collective of a training step).

    A rank whose rays all missed the tree has no gradient yet: it contributes zeros.
    """
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return None
    if _Overlap.reduced:        # summed range by range inside the backward pass
        _Overlap.reduced = False
        return None
    if tree.data.grad is None:
        tree.data.grad = torch.zeros_like(tree.data)
    return dist.all_reduce(tree.data.grad, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


def broadcast_tree(tree, src=0, group=None):
    """Replicate rank ``src``'s tree tensors (same shapes everywhere) to all ranks."""
    for t in (tree.data.data, tree.child, tree.parent_depth, tree.invradius, tree.offset,
              tree._n_internal, tree._n_free):
        dist.broadcast(t, src=src, group=group)
    tree._invalidate()


def gather_rows(local, n_total, group=None):
    """Reassemble per-rank row slices (as cut by ``shard_rows``) into the full tensor."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    parts = []
    for r in range(world):
        lo, hi = shard_bounds(n_total, r, world)
        parts.append(torch.empty((hi - lo, *local.shape[1:]), dtype=local.dtype,
                                 device=local.device))
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=0)
