"""Sparse N^3-tree (N = 2: octree) storage with CUDA point queries.

Drop-in for the reference's ``svox.N3Tree`` on the query / render path
(svox/svox.py:57-155 constructor and tensors, :208-272 ``forward``,
:636-705 ``refine``, :947-951 ``__getitem__``, :1015-1024 index packing,
:1067-1071 ``world2tree``, :1084-1103 ``_spec``).

Storage is three flat tensors, identical in name, shape and meaning to the
reference so that ``state_dict`` and checkpoints stay interchangeable:

* ``data``          ``(M, N, N, N, K)`` float32 ``nn.Parameter`` -- one record per slot,
* ``child``         ``(M, N, N, N)`` int32 -- 0 for a leaf, else ``child_node - node``,
* ``parent_depth``  ``(M, 2)`` int32 -- packed parent slot and depth (root: depth -1 ... 0).

Point queries on a CUDA tree run the ``query_vertical`` kernels of the
native library; there is no CPU implementation of the query in this
package (a CPU tree raises).
"""
import math
import weakref
from warnings import warn

import numpy as np
import torch
from torch import autograd, nn

from . import csrc as _C
from .formats import DataFormat, LocalIndex
from .view import N3TreeView

__all__ = ["N3Tree", "WeightAccumulator", "_QueryVerticalFunction"]


class _QueryVerticalFunction(autograd.Function):
    """Autograd boundary of the point query (svox/svox.py:38-54)."""

    @staticmethod
    def forward(ctx, data, tree_spec, indices):
        out, node_ids = _C.query_vertical(tree_spec, indices)
        ctx.mark_non_differentiable(node_ids)
        ctx.tree_spec = tree_spec
        ctx.save_for_backward(indices)
        return out, node_ids

    @staticmethod
    def backward(ctx, grad_out, dummy):
        # (clearing the gradient buffer on a second stream beside the forward query, as the
        # renderer does, was measured: no gain, both are bound by DRAM)
        if ctx.needs_input_grad[0]:
            return _C.query_vertical_backward(ctx.tree_spec, ctx.saved_tensors[0],
                                              grad_out.contiguous()), None, None
        return None, None, None


class N3Tree(nn.Module):
    def __init__(self, N=2, data_dim=None, depth_limit=10, init_reserve=1, init_refine=0,
                 geom_resize_fact=1.0, radius=0.5, center=(0.5, 0.5, 0.5), data_format="RGBA",
                 extra_data=None, device="cpu", dtype=torch.float32, map_location=None):
        super().__init__()
        assert N >= 2
        assert depth_limit >= 0
        if map_location is not None:
            warn("map_location has been renamed to device and may be removed")
            device = map_location
        assert dtype in (torch.float32, torch.float64), "Unsupported dtype"
        self.N = N
        self.data_format = DataFormat(data_format) if data_format is not None else None
        self.data_dim = data_dim
        self._maybe_auto_data_dim()

        # one node per cell of every level that init_refine will create
        init_reserve += sum((N ** i) ** 3 for i in range(1, init_refine + 1))

        self.register_parameter("data", nn.Parameter(
            torch.zeros(init_reserve, N, N, N, self.data_dim, dtype=dtype, device=device)))
        self.register_buffer("child", torch.zeros(init_reserve, N, N, N, dtype=torch.int32,
                                                  device=device))
        self.register_buffer("parent_depth", torch.zeros(init_reserve, 2, dtype=torch.int32,
                                                         device=device))
        self.register_buffer("_n_internal", torch.tensor(1, device=device))
        self.register_buffer("_n_free", torch.tensor(0, device=device))

        if isinstance(radius, (int, float)):
            radius = [radius] * 3
        radius = torch.tensor(radius, dtype=dtype, device=device)
        center = torch.tensor(list(center), dtype=dtype, device=device)
        self.register_buffer("invradius", 0.5 / radius)
        self.register_buffer("offset", 0.5 * (1.0 - center / radius))

        self.depth_limit = depth_limit
        self.geom_resize_fact = geom_resize_fact
        if extra_data is not None:
            assert isinstance(extra_data, torch.Tensor)
            self.register_buffer("extra_data", extra_data.to(dtype=dtype, device=device))
        else:
            self.extra_data = None

        self._ver = 0
        self._data_epoch = 0     # bumped by every write that goes through ``data.data``
        self._invalidate()
        self._lock_tree_structure = False
        self._weight_accum = None
        self._weight_accum_op = None
        self.refine(repeats=init_refine)

    # ------------------------------------------------------------------
    # Point assignment
    def set(self, indices, values, cuda=True):
        """Overwrite the leaf containing each point of ``indices`` ``(Q, 3)`` with its row of
        ``values`` ``(Q, K)`` (svox/svox.py:159-206).  Points that share a leaf race, as in
        the reference.  The tree must live on a CUDA device."""
        assert len(indices.shape) == 2
        assert not indices.requires_grad  # Grad wrt indices not supported
        assert not values.requires_grad  # Grad wrt values not supported
        if not cuda or not self.data.is_cuda:
            raise RuntimeError(
                "svox_b200 has no CPU assignment path: move the tree to a CUDA device "
                "(tree.cuda()) and call with cuda=True")
        dev, dt = self.data.device, self.data.dtype
        indices = indices.to(device=dev, dtype=dt).contiguous()
        values = values.to(device=dev, dtype=dt).contiguous()
        self._data_epoch += 1
        _C.assign_vertical(self._spec(), indices, values)

    # ------------------------------------------------------------------
    # Point query (hot path)
    def forward(self, indices, cuda=True, want_node_ids=False, world=True):
        """Values (and packed leaf ids) of the leaves containing ``indices`` ``(Q, 3)``.

        Differentiable w.r.t. ``data``.  Same contract as svox/svox.py:208-272;
        the tree must live on a CUDA device.
        """
        assert not indices.requires_grad  # Grad wrt indices not supported
        assert len(indices.shape) == 2
        if not cuda or not self.data.is_cuda:
            raise RuntimeError(
                "svox_b200 has no CPU query path: move the tree to a CUDA device "
                "(tree.cuda()) and call with cuda=True")
        result, node_ids = _QueryVerticalFunction.apply(self.data, self._spec(world), indices)
        return (result, node_ids) if want_node_ids else result

    def __getitem__(self, key):
        return N3TreeView(self, key)

    def __setitem__(self, key, val):
        N3TreeView(self, key).set(val)

    def snap(self, indices):
        return self[indices].corners

    # ------------------------------------------------------------------
    # Structure
    def refine(self, repeats=1, sel=None):
        """Split every selected leaf into N^3 children, ``repeats`` times.

        Node numbering is part of the contract (leaf ids returned by queries
        are ``node * N^3 + cell``): new nodes are appended in selector order,
        the default selector lists leaves in row-major ``(node, u, v, w)``
        order, and a repeat selects the new nodes' cells in the same order
        (svox/svox.py:636-705).  Children inherit the parent's record.
        Returns True iff ``data`` was re-allocated.
        """
        if self._lock_tree_structure:
            raise RuntimeError("Tree locked")
        n3 = self.N ** 3
        resized = False
        with torch.no_grad():
            slots = None
            for rep in range(repeats):
                filled = self.n_internal
                if slots is None:
                    if sel is None:
                        sel = tuple(self._all_leaves().T)
                    slots = self._pack_index(torch.stack(
                        [s.to(self.child.device).long() for s in sel], dim=-1))
                nodes = torch.div(slots, n3, rounding_mode="floor")
                ok = (self.parent_depth[nodes, 1] < self.depth_limit) & \
                     (self.child.view(-1)[slots] == 0)
                slots, nodes = slots[ok], nodes[ok]
                n_new = slots.numel()
                if n_new == 0:
                    return False
                grow = filled + n_new - self.capacity
                if grow > 0:
                    self._resize_add_cap(grow)
                    resized = True
                new_ids = torch.arange(filled, filled + n_new, device=slots.device)
                self.child[filled:filled + n_new] = 0
                self.child.view(-1)[slots] = (new_ids - nodes).to(torch.int32)
                flat = self.data.data.view(-1, self.data_dim)
                self.data.data[filled:filled + n_new] = flat[slots][:, None, None, None]
                self.parent_depth[filled:filled + n_new, 0] = slots.to(torch.int32)
                self.parent_depth[filled:filled + n_new, 1] = self.parent_depth[nodes, 1] + 1
                if rep < repeats - 1:
                    slots = (new_ids[:, None] * n3 +
                             torch.arange(n3, device=slots.device)[None]).reshape(-1)
                self._n_internal += n_new
        if repeats > 0:
            self._invalidate()
        return resized

    def check_integrity(self):
        """Structural invariants (as svox/svox.py:583-618); raises AssertionError."""
        n_int, n_free = self.n_internal, self._n_free.item()
        assert n_int - n_free > 0, "Tree has no root"
        assert self.data.shape[0] == self.capacity, "Data capacity mismatch"
        assert self.child.shape[0] == self.capacity, "Child capacity mismatch"
        assert (self.parent_depth[0] == 0).all(), "Node at index 0 must be root"
        live = (self.parent_depth[:n_int, 0] != -1).nonzero().reshape(-1)
        links = self.child[live]
        assert (links >= 0).all(), "Nodes not topologically sorted"
        target = links.long() + live[:, None, None, None]
        assert target.max() < n_int, "Tree has an out-of-bounds child link"
        assert (self.parent_depth[target.reshape(-1), 0] != -1).all(), \
            "Tree has a child link to a deleted node"
        rest = live[live != 0]
        if rest.numel() == 0:
            return True
        pslot = self.parent_depth[rest, 0].long()
        assert pslot.min() >= 0 and pslot.max() < n_int * self.N ** 3, "Parent link out-of-bounds"
        pnode = torch.div(pslot, self.N ** 3, rounding_mode="floor")
        assert (pnode + self.child.view(-1)[pslot] == rest).all(), \
            "parent->child cycle consistency failed"
        return True

    # ------------------------------------------------------------------
    # Sizes
    @property
    def n_leaves(self):
        return self._all_leaves().shape[0]

    @property
    def n_internal(self):
        return self._n_internal.item()

    @property
    def capacity(self):
        return self.parent_depth.shape[0]

    @property
    def max_depth(self):
        return torch.max(self.depths).item()

    @property
    def ndim(self):
        return 2

    @property
    def shape(self):
        return torch.Size((self.n_leaves, self.data_dim))

    def size(self, dim):
        return self.data_dim if dim == 1 else self.n_leaves

    def numel(self):
        return self.data_dim * self.n_leaves

    def __len__(self):
        return self.n_leaves

    def __repr__(self):
        return (f"svox.N3Tree(N={self.N}, data_dim={self.data_dim}, "
                f"depth_limit={self.depth_limit}, "
                f"capacity:{self.n_internal - self._n_free.item()}/{self.capacity}, "
                f"data_format:{self.data_format or 'RGBA'})")

    # ------------------------------------------------------------------
    # Persistence (svox/svox.py:835-865, 899-938): same npz keys, data as fp16
    def accumulate_weights(self, op: str = "sum"):
        """Begin weight accumulation (svox/svox.py:810-832): forward renders inside the
        ``with`` block add (``op="sum"``) every contributing sample's weight to its leaf,
        or keep the largest (``op="max"``).

            with tree.accumulate_weights() as accum:
                renderer(rays)
            w = accum()          # (n_leaves,), in the order of ``tree.values``
        """
        return WeightAccumulator(self, op)

    # The checkpoint is a flat npz whose keys, dtypes and meanings are the reference's file
    # format (svox/svox.py:835-865, 899-938): (key, how to read it off a tree, how to put it
    # back).  ``data`` is stored as float16; ``invradius3`` replaced a scalar ``invradius`` in
    # older files; ``n_free``, ``data_format`` and ``extra_data`` may be absent.
    _NPZ_FIELDS = (
        ("data_dim", lambda t: t.data_dim, lambda t, v, dev: setattr(t, "data_dim", int(v))),
        ("child", lambda t: t.child.cpu(),
         lambda t, v, dev: setattr(t, "child", torch.from_numpy(v).to(dev))),
        ("parent_depth", lambda t: t.parent_depth.cpu(),
         lambda t, v, dev: setattr(t, "parent_depth", torch.from_numpy(v).to(dev))),
        ("n_internal", lambda t: t._n_internal.cpu().item(),
         lambda t, v, dev: t._n_internal.fill_(v.item())),
        ("n_free", lambda t: t._n_free.cpu().item(), lambda t, v, dev: t._n_free.fill_(v.item())),
        ("invradius3", lambda t: t.invradius.cpu(),
         lambda t, v, dev: setattr(t, "invradius",
                                   torch.from_numpy(v.astype(np.float32)).to(dev))),
        ("offset", lambda t: t.offset.cpu(),
         lambda t, v, dev: setattr(t, "offset", torch.from_numpy(v.astype(np.float32)).to(dev))),
        ("depth_limit", lambda t: t.depth_limit,
         lambda t, v, dev: setattr(t, "depth_limit", int(v))),
        ("geom_resize_fact", lambda t: t.geom_resize_fact,
         lambda t, v, dev: setattr(t, "geom_resize_fact", float(v))),
        ("data", lambda t: t.data.data.half().cpu().numpy(), None),     # handled by load()
        ("data_format", lambda t: None if t.data_format is None else repr(t.data_format),
         lambda t, v, dev: setattr(t, "data_format", DataFormat(v.item()))),
        ("extra_data", lambda t: None if t.extra_data is None else t.extra_data.cpu(),
         lambda t, v, dev: setattr(t, "extra_data", torch.from_numpy(v).to(dev))),
    )

    def save(self, path, shrink=True, compress=True):
        """Write the tree as an npz in the reference's checkpoint format (``data`` as fp16)."""
        if shrink:
            self.shrink_to_fit()
        blob = {}
        for key, read, _ in self._NPZ_FIELDS:
            value = read(self)
            if value is not None:
                blob[key] = value
        (np.savez_compressed if compress else np.savez)(path, **blob)

    @classmethod
    def load(cls, path, device="cpu", dtype=torch.float32, map_location=None):
        """Read a checkpoint written by this package or by the reference."""
        if map_location is not None:
            warn("map_location has been renamed to device and may be removed")
            device = map_location
        assert dtype in (torch.float32, torch.float64), "Unsupported dtype"
        z = np.load(path)
        tree = cls(dtype=dtype, device=device)
        tree.data_format = tree.extra_data = None
        tree._n_free.zero_()
        for key, _, write in cls._NPZ_FIELDS:
            if write is not None and key in z.files:
                write(tree, z[key], device)
        if "invradius3" not in z.files:                  # files older than per-axis radii
            tree.invradius.fill_(z["invradius"].item())
        tree.N = tree.child.shape[-1]
        tree.data = nn.Parameter(torch.from_numpy(z["data"].astype(np.float32)).to(
            device=device, dtype=dtype))
        tree._invalidate()
        return tree

    # ------------------------------------------------------------------
    # Coarsening: frontier nodes (all of whose cells are leaves), merging them back into
    # their parents, and compaction (svox/svox.py:436-580, 620-632, 745-788).
    @property
    def _frontier(self):
        """Ids of the live nodes all of whose cells are leaves, ascending."""
        if self._last_frontier is None:
            n = self.n_internal
            only_leaves = (self.child[:n] == 0).flatten(1).all(dim=1)
            alive = self.parent_depth[:n, 0] != -1
            self._last_frontier = torch.nonzero(only_leaves & alive).flatten()
        return self._last_frontier

    @property
    def n_frontier(self):
        return self._frontier.shape[0]

    @property
    def frontier_depth(self):
        return self.parent_depth[self._frontier, 1]

    def reduce_frontier(self, op=torch.mean, dim=None, grad=False):
        """``op`` over the N^3 leaf records of every frontier node: ``op(x, dim=1)`` with ``x``
        of shape ``(n_frontier, N^3, data_dim)`` (or the selected channels ``dim``)."""
        src = self.data if grad else self.data.data
        x = src[self._frontier].reshape(-1, self.N ** 3, self.data_dim)
        return op(x if dim is None else x[..., dim], dim=1)

    def max_frontier(self, dim=None, grad=False):
        return self.reduce_frontier(lambda x, dim: torch.max(x, dim=dim)[0], dim=dim, grad=grad)

    def diam_frontier(self, dim=None, grad=False, scale=1.0):
        """Largest pairwise distance between the leaf records of every frontier node."""
        def diameter(x, dim):
            if x.ndim == 2:
                x = x[:, :, None]
            pair = torch.cdist(x * scale, x * scale)          # (B, N^3, N^3)
            return pair.flatten(1).max(dim=1)[0]
        return self.reduce_frontier(diameter, dim=dim, grad=grad)

    def merge(self, frontier_sel=None, op=torch.mean):
        """Turn the selected frontier nodes back into leaves of their parents, whose record
        becomes ``op`` over the children's.  The freed nodes stay in the arrays (marked with
        -1) until ``shrink_to_fit``.  Returns False if nothing was selected."""
        if self._lock_tree_structure:
            raise RuntimeError("Tree locked")
        if self.n_internal - self._n_free.item() <= 1:
            raise RuntimeError("Cannot merge root node")
        nodes = self._frontier if frontier_sel is None else self._frontier[frontier_sel]
        nodes = nodes.reshape(-1)
        if nodes.numel() == 0:
            return False
        with torch.no_grad():
            merged = op(self.data.data[nodes].reshape(-1, self.N ** 3, self.data_dim), dim=1)
            if isinstance(merged, tuple):                 # torch.max / torch.min return pairs
                merged = merged[0]
            parent_slot = self.parent_depth[nodes, 0].long()
            self.data.data.view(-1, self.data_dim)[parent_slot] = merged
            self.child.view(-1)[parent_slot] = 0
            self.parent_depth[nodes] = -1
            self.child[nodes] = -1
            self._n_free += nodes.shape[0]
        self._invalidate()
        return True

    # ------------------------------------------------------------------
    # Copies and channel layout (svox/svox.py:286-430)
    def partial(self, data_sel=None, data_format=None, dtype=None, device=None):
        """Copy of the tree that keeps only the channels ``data_sel`` of every record (all by
        default), e.g. ``tree.partial(-1)`` for the densities alone.  As in the reference the
        copy carries THIS tree's ``data_format`` object; ``data_format`` only has to name a
        format the new channel count is valid for (``"RGBA"`` accepts any)."""
        device = self.data.device if device is None else device
        dtype = self.data.dtype if dtype is None else dtype
        channels = None
        if data_sel is not None:
            channels = torch.arange(self.data_dim)[data_sel].reshape(-1)
        other = N3Tree(N=self.N,
                       data_dim=self.data_dim if channels is None else channels.numel(),
                       data_format=data_format or str(self.data_format),
                       depth_limit=self.depth_limit, geom_resize_fact=self.geom_resize_fact,
                       dtype=dtype, device=device)

        def moved(x):
            return x.detach().to(device=device, copy=True)

        for name in ("invradius", "offset", "child", "parent_depth", "_n_internal", "_n_free"):
            setattr(other, name, moved(getattr(self, name)))
        other.extra_data = None if self.extra_data is None else moved(self.extra_data)
        other.data_format = self.data_format
        values = self.data.data if channels is None else \
            self.data.data[..., channels.to(self.data.device)]
        other.data = nn.Parameter(moved(values).to(dtype).contiguous())
        other._invalidate()
        return other

    def clone(self, device=None):
        """Deep copy, optionally onto another device."""
        return self.partial(device=device)

    def expand(self, data_format, data_dim=None, remap=None):
        """Change the record layout to ``data_format`` (more or fewer basis functions per
        colour channel).  ``remap`` lists, for the smaller of the two layouts, the channel of
        the larger one that each of its channels corresponds to; by default colour channel c's
        basis function i stays basis function i and the density stays last.  New channels are
        zero.  Replaces the ``data`` parameter: optimizers have to be rebuilt."""
        assert isinstance(data_format, str), "Please specify valid data format"
        old_format, old_dim = self.data_format, self.data_dim
        self.data_format = DataFormat(data_format)
        self.data_dim = data_dim
        self._maybe_auto_data_dim()
        small, large = sorted((old_dim, self.data_dim))
        if remap is None:
            fmt_small, fmt_large = (old_format, self.data_format) if old_dim <= self.data_dim \
                else (self.data_format, old_format)
            if old_format is None or self.data_format.format == DataFormat.RGBA:
                remap = torch.cat([torch.arange(small - 1), torch.tensor([large - 1])])
            else:
                assert self.data_format.basis_dim >= 1, \
                    "Please manually specify data_dim for expand()"
                n_small = max(fmt_small.basis_dim, 1)
                n_large = max(fmt_large.basis_dim, 1)
                fn = torch.arange(n_small)
                remap = torch.cat([fn, n_large + fn, 2 * n_large + fn, torch.tensor([large - 1])])
        remap = torch.as_tensor(remap, device=self.data.device)
        old = self.data.data
        new = torch.zeros((*old.shape[:-1], self.data_dim), dtype=old.dtype, device=old.device)
        if self.data_dim < old_dim:
            new[:] = old[..., remap]
        else:
            new[..., remap] = old
        self.data = nn.Parameter(new)
        self._invalidate()

    def shrink(self, data_format, data_dim=None, remap=None):
        """Alias of :meth:`expand`, which goes both ways."""
        self.expand(data_format, data_dim, remap)

    # In-place arithmetic on all leaves
    def __iadd__(self, val):
        self[:] += val
        return self

    def __isub__(self, val):
        self[:] -= val
        return self

    def __imul__(self, val):
        self[:] *= val
        return self

    def __itruediv__(self, val):
        self[:] /= val
        return self

    __idiv__ = __itruediv__

    def _make_val_tensor(self, val):
        """``val`` as a ``(1 or B, data_dim)`` tensor on the tree's device."""
        t = torch.as_tensor(val, dtype=self.data.dtype, device=self.data.device)
        while t.dim() < 2:
            t = t[None]
        if t.shape[-1] == 1:
            return t.expand(-1, self.data_dim).contiguous()
        assert t.shape[-1] == self.data_dim
        return t

    def shrink_to_fit(self):
        """Drop unused capacity and the nodes freed by ``merge``: the surviving nodes move up
        in order, links and parent slots are renumbered.  Re-creates the ``data`` parameter
        (an optimizer holding the old one must be rebuilt)."""
        if self._lock_tree_structure:
            raise RuntimeError("Tree locked")
        n_int, n_free = self.n_internal, int(self._n_free.item())
        new_cap = n_int - n_free
        if new_cap >= self.capacity:
            return False
        with torch.no_grad():
            if n_free == 0:
                keep = slice(0, new_cap)
            else:
                n3 = self.N ** 3
                dead = self.parent_depth[:n_int, 0] == -1
                new_id = torch.cumsum(~dead, dim=0) - 1          # id of a survivor after the move
                keep = torch.nonzero(~dead).flatten()
                # every survivor but the root: its parent's link and its own parent slot
                kids = keep[keep != 0]
                pslot = self.parent_depth[kids, 0].long()
                pnode = torch.div(pslot, n3, rounding_mode="floor")
                self.child.view(-1)[pslot] = (new_id[kids] - new_id[pnode]).to(torch.int32)
                self.parent_depth[kids, 0] = (new_id[pnode] * n3 + pslot % n3).to(torch.int32)
                self._n_internal.fill_(new_cap)
                self._n_free.zero_()
            self.data = nn.Parameter(self.data.data[keep].clone())
            self.child = self.child[keep].clone()
            self.parent_depth = self.parent_depth[keep].clone()
        self._invalidate()
        return True

    # ------------------------------------------------------------------
    # Internal utilities
    def _pack_index(self, txyz):
        N = self.N
        return txyz[:, 0] * (N ** 3) + txyz[:, 1] * (N ** 2) + txyz[:, 2] * N + txyz[:, 3]

    def _unpack_index(self, flat):
        N = self.N
        w = flat % N
        v = torch.div(flat, N, rounding_mode="floor") % N
        u = torch.div(flat, N * N, rounding_mode="floor") % N
        node = torch.div(flat, N ** 3, rounding_mode="floor")
        return torch.stack((node, u, v, w), dim=-1)

    def _resize_add_cap(self, cap_needed):
        cap_needed = max(cap_needed, int(self.capacity * (self.geom_resize_fact - 1.0)))

        def grow(t):
            pad = torch.zeros((cap_needed, *t.shape[1:]), dtype=t.dtype, device=t.device)
            return torch.cat((t, pad), dim=0)

        self.data = nn.Parameter(grow(self.data.data))
        self.child = grow(self.child)
        self.parent_depth = grow(self.parent_depth)

    def _all_leaves(self):
        if self._last_all_leaves is None:
            self._last_all_leaves = (self.child[:self.n_internal] == 0).nonzero(
                as_tuple=False).cpu()
        return self._last_all_leaves

    def _calc_corners(self, nodes, cuda=True):
        """Lower corner of each ``(node, u, v, w)`` cell in tree-local coordinates
        (svox/svox.py:990-1012): the native kernel on a CUDA tree, tensor ops otherwise."""
        if self.data.is_cuda and cuda:
            nodes = nodes.to(device=self.data.device, dtype=torch.int64).contiguous()
            return _C.calc_corners(self._spec(), nodes)
        nodes = nodes.to(self.parent_depth.device).long()
        out = torch.zeros(nodes.shape[0], 3, device=nodes.device, dtype=self.data.dtype)
        alive = torch.arange(nodes.shape[0], device=nodes.device)
        cur = nodes
        while alive.numel():
            out[alive] = (out[alive] + cur[:, 1:].to(out.dtype)) / self.N
            up = cur[:, 0] != 0
            alive, cur = alive[up], cur[up]
            if alive.numel():
                cur = self._unpack_index(self.parent_depth[cur[:, 0], 0].long())
        return out.to(self.data.device)

    def world2tree(self, indices):
        return torch.addcmul(self.offset, indices, self.invradius)

    def tree2world(self, indices):
        return (indices - self.offset) / self.invradius

    def _invalidate(self):
        self._ver += 1
        self._data_epoch += 1
        self._last_all_leaves = None
        self._last_frontier = None

    def _spec(self, world=True):
        """Pack the tensors for the native library (svox/svox.py:1084-1103)."""
        spec = _C.TreeSpec()
        spec._owner = weakref.ref(self)
        spec.data = self.data
        spec.child = self.child
        spec.parent_depth = self.parent_depth
        dev, dt = self.data.device, self.data.dtype
        spec.extra_data = self.extra_data if self.extra_data is not None else \
            torch.empty((0, 0), dtype=dt, device=dev)
        if world:
            spec.offset, spec.scaling = self.offset, self.invradius
        else:
            spec.offset = torch.zeros(3, dtype=dt, device=dev)
            spec.scaling = torch.ones(3, dtype=dt, device=dev)
        spec._weight_accum = self._weight_accum if self._weight_accum is not None else \
            torch.empty(0, dtype=dt, device=dev)
        spec._weight_accum_max = (self._weight_accum_op == "max")
        return spec

    def _maybe_auto_data_dim(self):
        fmt = self.data_format
        if fmt is not None and fmt.data_dim is not None:
            if self.data_dim is None:
                self.data_dim = fmt.data_dim
            else:
                assert fmt.data_dim == self.data_dim, "data_dim invalid for given data format"
        elif self.data_dim is None:
            self.data_dim = 4  # legacy RGBA default

    @classmethod
    def from_grid(cls, grid, *args, **kwargs):
        D = grid.shape[0]
        assert grid.ndim == 4 and grid.shape[1] == D and grid.shape[2] == D, \
            "Grid must be a 4D array with first 3 dims equal"
        logd = int(math.log2(D))
        assert 2 ** logd == D, "Grid size must be power of 2"
        kwargs["init_refine"] = logd - 1
        tree = cls(*args, **kwargs)
        tree.set_grid(grid)
        return tree

    def set_grid(self, grid):
        D = grid.shape[0]
        assert grid.ndim == 4 and grid.shape[1] == D and grid.shape[2] == D and \
            grid.shape[-1] == self.data_dim
        arr = (torch.arange(D) + 0.5) / D
        xyz = torch.stack(torch.meshgrid(arr, arr, arr, indexing="ij"), -1).reshape(-1, 3)
        self[LocalIndex(xyz.to(self.data.device))] = grid.reshape(-1, self.data_dim).to(
            self.data.device)


def _install_view_redirects():
    """``tree.depths`` == ``tree[:].depths`` etc. (svox/svox.py:1106-1123)."""
    props = ["depths", "lengths", "lengths_local", "corners", "corners_local", "values",
             "values_local"]
    funcs = ["sample", "sample_local", "aux", "normal_", "clamp_", "uniform_", "relu_",
             "sigmoid_", "nan_to_num_"]

    def add_func(name):
        setattr(N3Tree, name, lambda self, *a, **k: getattr(self[:], name)(*a, **k))

    def add_prop(name):
        setattr(N3Tree, name, property(lambda self: getattr(self[:], name)))

    for n in funcs:
        add_func(n)
    for n in props:
        add_prop(n)


_install_view_redirects()


class WeightAccumulator:
    """Context manager behind ``N3Tree.accumulate_weights`` (svox/svox.py:1136-1161)."""

    def __init__(self, tree, op):
        assert op in ["sum", "max"], "Unsupported accumulation"
        self.tree = tree
        self.op = op

    def __enter__(self):
        self.tree._lock_tree_structure = True
        self.tree._weight_accum = torch.zeros(self.tree.child.shape, dtype=self.tree.data.dtype,
                                              device=self.tree.data.device)
        self.tree._weight_accum_op = self.op
        self.weight_accum = self.tree._weight_accum
        return self

    def __exit__(self, type, value, traceback):
        self.tree._weight_accum = None
        self.tree._weight_accum_op = None
        self.tree._lock_tree_structure = False

    @property
    def value(self):
        return self.weight_accum

    def __call__(self):
        return self.tree[:].aux(self.weight_accum)
