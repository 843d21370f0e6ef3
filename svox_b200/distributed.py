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
           "gather_rows", "overlap_grad_allreduce", "MulticastGradient"]


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
    reduced = 0       # backward passes since the last allreduce_grad whose gradient left the
    backwards = 0     # renderer already summed / all of them that went through the hook

    @classmethod
    def on_part(cls, rows):
        if rows.numel() == 0:       # the same ranges are empty on every rank
            return
        cls.works.append(dist.all_reduce(rows, op=dist.ReduceOp.SUM, group=cls.group,
                                         async_op=True))

    @classmethod
    def on_done(cls):
        for w in cls.works:
            w.wait()            # the current stream waits for the collective's stream
        cls.works = []
        cls.reduced += 1


def overlap_grad_allreduce(n_parts=8, group=None, reserve_sms=16):
    """Overlap the all-reduce of ``data.grad`` with its computation.

    The replay backward of the renderer produces the gradient leaf range by leaf range;
    with this switched on, the rows of a finished range are all-reduced (asynchronously, on
    the backend's stream) while the next range is computed, and ``reserve_sms`` SMs are left
    to the collective's kernel.  ``allreduce_grad`` then finds the gradient already summed
    and does nothing.  The ranges depend on the tree's size alone and the host never looks
    at device results on this route (an item log that turns out too small is handled on the
    device), so every rank issues the same collectives in the same order.  Backward passes
    that do not replay (thresholds on, ``data`` edited since the forward) leave their
    gradient to ``allreduce_grad``.  ``n_parts=0`` switches it off.
    Every rank must make the same call.
    """
    from . import render
    if not n_parts or not (dist.is_available() and dist.is_initialized()) \
            or dist.get_world_size(group) == 1:
        render.GRAD_PARTS = None
        return
    _Overlap.group = group
    _Overlap.works = []
    _Overlap.reduced = 0
    render.GRAD_PARTS = (int(n_parts), _Overlap.on_part, _Overlap.on_done,
                         int(reserve_sms) if n_parts > 1 else 0)   # one part: nothing overlaps


class MulticastGradient:
    """``tree.data.grad`` kept in symmetric memory and summed across the GPUs of one NVSwitch
    domain by the switch itself (``svoxb_allreduce_multimem``) instead of an NCCL ring.

    While ``enabled``, the renderer's training step accumulates its gradient into this
    buffer (a fresh view of it per step, which autograd adopts as ``data.grad`` without a
    copy), and ``allreduce_grad(tree)`` sums it in place: a barrier across the ranks, the
    kernel, a second barrier, all on the current stream; the host waits for nothing.
    One gradient is alive at a time: drop ``data.grad`` (``zero_grad(set_to_none=True)``)
    before the next step's forward.  Every rank must construct it, in the same order.
    Raises ``RuntimeError`` where the GPUs offer no multicast memory.
    """
    active = None

    def __init__(self, tree, group=None):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.shape = tuple(tree.data.shape)
        n = tree.data.numel()
        self.n, self.padded = n, (n + 3) // 4 * 4
        self.flat = symm.empty(self.padded, dtype=torch.float32, device=tree.data.device)
        self.handle = symm.rendezvous(self.flat, self.group)
        if not self.handle.multicast_ptr:
            raise RuntimeError("these GPUs offer no multicast memory")
        self.flat.zero_()
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)

    def view(self, like=None):
        return self.flat[:self.n].view(self.shape)

    def enable(self):
        from . import render
        render.GRAD_BUFFER = self.view
        MulticastGradient.active = self

    @staticmethod
    def disable():
        from . import render
        render.GRAD_BUFFER = None
        MulticastGradient.active = None

    def owns(self, t):
        return t is not None and t.untyped_storage().data_ptr() == \
            self.flat.untyped_storage().data_ptr()

    def allreduce_(self):
        from . import csrc
        self.handle.barrier(channel=0)      # every rank's gradient is complete
        csrc.allreduce_multimem(self.handle.multicast_ptr, self.padded, self.rank, self.world)
        self.handle.barrier(channel=1)      # every rank's slice of sums has been written


def allreduce_grad(tree, group=None, async_op=False):
    """Sum ``tree.data.grad`` over all ranks (the one collective of a training step).

    A rank whose rays all missed the tree has no gradient yet: it contributes zeros.
    With ``overlap_grad_allreduce`` on, a step with ONE backward pass arrives here already
    summed.  A step that accumulated several backward passes into ``data.grad`` cannot be
    told apart element by element, so that combination is refused: switch the overlap off
    when accumulating gradients.
    """
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return None
    reduced, _Overlap.reduced = _Overlap.reduced, 0
    if reduced == 1:            # summed range by range inside the backward pass
        return None
    if reduced > 1:
        raise RuntimeError(
            "allreduce_grad: several backward passes were reduced inside the backward and "
            "accumulated into data.grad; call allreduce_grad after each backward, or switch "
            "overlap_grad_allreduce off when accumulating gradients")
    mc = MulticastGradient.active
    if mc is not None:
        if tree.data.grad is None:
            mc.flat.zero_()
            tree.data.grad = mc.view()
        if mc.owns(tree.data.grad):
            mc.allreduce_()
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
