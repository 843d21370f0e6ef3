"""B200-native implementation of svox's octree query and volume rendering path.

Use as a drop-in: ``import svox_b200 as svox``.
"""
from .formats import DataFormat, LocalIndex
from .view import N3TreeView
from .tree import N3Tree
from .render import VolumeRenderer, NDCConfig, Rays

__version__ = "0.1.0"
__all__ = ["N3Tree", "N3TreeView", "VolumeRenderer", "NDCConfig", "Rays", "LocalIndex",
           "DataFormat"]
