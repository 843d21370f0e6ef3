"""Module alias: ``svox.svox`` names of the reference (svox/svox.py)."""
from .tree import N3Tree, _QueryVerticalFunction  # noqa: F401
