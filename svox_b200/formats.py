"""Leaf record formats and the local-coordinate key wrapper.

Behaviour follows the reference's ``DataFormat`` and ``LocalIndex``
(svox/helpers.py:376-424): a format string is letters followed by an
optional integer, the integer is the number of basis functions per colour
channel, and a leaf record holds ``3 * basis_dim + 1`` floats laid out
channel-major with the density last.
"""

__all__ = ["DataFormat", "LocalIndex"]

_NAMES = {"RGBA": 0, "SH": 1, "SG": 2, "ASG": 3}


class DataFormat:
    RGBA = 0
    SH = 1
    SG = 2
    ASG = 3

    def __init__(self, txt):
        txt = str(txt)
        # Split at the first character that is not a letter; what follows must
        # parse as an integer (so "S4H" raises ValueError, as in the reference).
        first = next((i for i, ch in enumerate(txt) if not ch.isalpha()), len(txt))
        head, digits = txt[:first], txt[first:]
        if digits:
            self.basis_dim = int(digits)
            assert self.basis_dim > 0, "data_format basis_dim must be positive"
            self.data_dim = 3 * self.basis_dim + 1
            self.format = _NAMES.get(head, DataFormat.RGBA)
            if self.format == DataFormat.SH:
                root = int(self.basis_dim ** 0.5)
                assert root * root == self.basis_dim, "SH basis dim must be square number"
                assert self.basis_dim <= 25, "SH only supported up to basis_dim 25"
        else:
            self.format = DataFormat.RGBA
            self.basis_dim = -1
            self.data_dim = None

    def __repr__(self):
        name = {v: k for k, v in _NAMES.items()}[self.format]
        return name + (str(self.basis_dim) if self.basis_dim >= 0 else "")

    def __eq__(self, other):
        return (isinstance(other, DataFormat) and self.format == other.format
                and self.basis_dim == other.basis_dim)

    def __hash__(self):
        return hash((self.format, self.basis_dim))


class LocalIndex:
    """Marks a ``(B, 3)`` key as tree-local ``[0, 1]^3`` coordinates: ``tree[LocalIndex(p)]``."""

    def __init__(self, val):
        self.val = val
