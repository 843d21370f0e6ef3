"""Tensor-like view onto a set of leaves of an :class:`N3Tree`.

Mirrors the behaviour of the reference's ``N3TreeView``
(svox/helpers.py:27-359).  A view stores an advanced-indexing key
``(node, u, v, w[, channel])`` into ``tree.data``; the ``(B, 3)`` point key
(``tree[points]``) is the branch on the query hot path: it runs the
``query_vertical`` kernel and unpacks the returned leaf ids
(svox/helpers.py:44-50).
"""
import torch

from .formats import LocalIndex

__all__ = ["N3TreeView"]


class N3TreeView:
    def __init__(self, tree, key):
        self.tree = tree
        self.single_key = False
        self._packed_ids = None
        self._value = None
        local = False

        if isinstance(key, tuple) and len(key) >= 3:
            # tree[x, y, z[, c]]: one world point, optional channel selector
            point = torch.tensor(key[:3], dtype=tree.data.dtype,
                                 device=tree.data.device).reshape(1, 3)
            key = (point, *key[3:]) if len(key) > 3 else point

        extra = key[1:] if isinstance(key, tuple) else ()
        leaf_key = key[0] if isinstance(key, tuple) else key
        if isinstance(leaf_key, LocalIndex):
            leaf_key, local = leaf_key.val, True

        if torch.is_tensor(leaf_key) and leaf_key.ndim == 2 and leaf_key.shape[1] == 3:
            # (B, 3) points -> leaves containing them (the query hot path)
            if leaf_key.dtype != tree.data.dtype:
                leaf_key = leaf_key.to(dtype=tree.data.dtype)
            _, ids = tree.forward(leaf_key, want_node_ids=True, world=not local)
            self._packed_ids = ids.clone()
            leaf_node = tuple(tree._unpack_index(ids.clone()).T)
        else:
            if isinstance(leaf_key, int):
                leaf_key = torch.tensor([leaf_key], device=tree.data.device)
                self.single_key = True
            leaf_node = tuple(tree._all_leaves()[leaf_key].T)
        self.key = (*leaf_node, *extra)
        self._tree_ver = tree._ver

    # -- helpers ---------------------------------------------------------
    def _check_ver(self):
        if self.tree._ver > self._tree_ver:
            self.key = self._packed_ids = None
            raise RuntimeError("N3TreeView has been invalidated because tree "
                               "data layout has changed")

    def _require_subindex(self):
        return (len(self.key) == 5 and not isinstance(self.key[-1], (slice, int)))

    def _dev_key(self, n):
        dev = self.tree.data.device
        return tuple(k.to(dev) if torch.is_tensor(k) else k for k in self.key[:n])

    def _gather(self, arr):
        if self._require_subindex():
            return arr[self._dev_key(4)][..., self.key[-1]]
        return arr[self._dev_key(len(self.key))]

    def _indexer(self):
        return torch.stack(self.key[:4], dim=-1)

    def _unique_node_key(self):
        if self._packed_ids is None:
            return self.key[:4]
        return tuple(self.tree._unpack_index(torch.unique(self._packed_ids)).T)

    # -- values ----------------------------------------------------------
    @property
    def values(self):
        """Values of the selected leaves, differentiable: ``(n_leaves, data_dim)``."""
        self._check_ver()
        ret = self._gather(self.tree.data)
        return ret[0] if self.single_key else ret

    @property
    def values_nograd(self):
        self._check_ver()
        ret = self._gather(self.tree.data.data)
        return ret[0] if self.single_key else ret

    def set(self, value):
        self._check_ver()
        if isinstance(value, N3TreeView):
            value = value.values_nograd
        data = self.tree.data.data
        # autograd's version counter does not see writes through ``.data``: count them, so
        # that a backward whose forward ran before this edit recomputes from the new values
        self.tree._data_epoch += 1
        if self._require_subindex():
            k4 = self._dev_key(4)
            tmp = data[k4]
            tmp[..., self.key[-1]] = value
            data[k4] = tmp
        else:
            data[self._dev_key(len(self.key))] = value

    def aux(self, arr):
        """Index an auxiliary ``(capacity, N, N, N, ...)`` array with this view."""
        return self._gather(arr)

    def refine(self, repeats=1):
        self._check_ver()
        return self.tree.refine(repeats, sel=self._unique_node_key())

    # -- geometry --------------------------------------------------------
    @property
    def depths(self):
        """Leaf depths (root = -1, its children = 0, ...): ``(n_leaves,)`` int32."""
        self._check_ver()
        pd = self.tree.parent_depth
        return pd[self.key[0].to(pd.device), 1]

    @property
    def lengths_local(self):
        self._check_ver()
        return self.tree.N ** (-self.depths.float() - 1.0)

    @property
    def lengths(self):
        self._check_ver()
        return self.lengths_local[:, None] / self.tree.invradius

    @property
    def corners_local(self):
        self._check_ver()
        return self.tree._calc_corners(self._indexer())

    @property
    def corners(self):
        self._check_ver()
        return (self.corners_local - self.tree.offset) / self.tree.invradius

    def sample_local(self, n_samples):
        corn, length = self.corners_local, self.lengths_local
        u = torch.rand((corn.shape[0], n_samples, 3), device=length.device, dtype=length.dtype)
        return corn[:, None] + u * length[:, None, None]

    def sample(self, n_samples, device=None):
        device = device or self.tree.data.device
        corn, length = self.corners.to(device), self.lengths.to(device)
        u = torch.rand((corn.shape[0], n_samples, 3), device=device, dtype=length.dtype)
        return corn[:, None] + u * length[:, None]

    # -- in-place conveniences --------------------------------------------
    def normal_(self, mean=0.0, std=1.0):
        self.set(torch.randn_like(self.values_nograd) * std + mean)

    def uniform_(self, min=0.0, max=1.0):
        self.set(torch.rand_like(self.values_nograd) * (max - min) + min)

    def clamp_(self, min=None, max=None):
        self.set(torch.clamp(self.values_nograd, min, max))

    def relu_(self):
        self.set(torch.relu(self.values_nograd))

    def sigmoid_(self):
        self.set(torch.sigmoid(self.values_nograd))

    def nan_to_num_(self, inf_val=2e4):
        self.set(torch.nan_to_num(self.values_nograd, nan=0.0, posinf=inf_val, neginf=-inf_val))

    def __setitem__(self, key, value):
        val = self.values_nograd
        val[key] = value
        self.set(val)

    # -- tensor protocol ---------------------------------------------------
    @property
    def shape(self):
        return self.values_nograd.shape

    @property
    def ndim(self):
        return 2

    def __repr__(self):
        return "N3TreeView(" + repr(self.values) + ")"

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        args = [a.values if isinstance(a, N3TreeView) else a for a in args]
        return func(*args, **(kwargs or {}))


def _forward_to_values():
    nograd = ["__floordiv__", "__mod__", "__eq__", "__ne__", "__ge__", "__gt__", "__le__",
              "__lt__", "__floor__", "__ceil__", "__round__", "item", "size", "dim", "numel"]
    grad = ["__add__", "__mul__", "__sub__", "__truediv__", "__radd__", "__rsub__", "__rmul__",
            "__abs__", "__pos__", "__neg__", "__len__", "clamp", "clamp_max", "clamp_min",
            "relu", "sigmoid", "max", "min", "mean", "sum", "__getitem__"]

    def bind(name, use_grad):
        def method(self, *args, **kwargs):
            src = self.values if use_grad else self.values_nograd
            return getattr(src, name)(*args, **kwargs)
        method.__name__ = name
        setattr(N3TreeView, name, method)

    for n in nograd:
        bind(n, False)
    for n in grad:
        bind(n, True)


_forward_to_values()
