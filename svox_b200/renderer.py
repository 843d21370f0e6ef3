"""Module alias: ``svox.renderer`` names of the reference (svox/renderer.py)."""
from .render import (VolumeRenderer, NDCConfig, Rays, _VolumeRenderFunction,  # noqa: F401
                     _VolumeRenderImageFunction, _rays_spec_from_rays, _make_camera_spec)
