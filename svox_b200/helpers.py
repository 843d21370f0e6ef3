"""Module alias: ``svox.helpers`` names of the reference (svox/helpers.py)."""
from .formats import DataFormat, LocalIndex  # noqa: F401
from .view import N3TreeView  # noqa: F401
