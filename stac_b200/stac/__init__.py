"""Drop-in replacements of the reference's ``stac`` package exports (stac/__init__.py:3-11)."""

from .kv_manager import KVManager
from .h2o import HeavyHittersKV
from .stac_voxel import STACVoxelKV

__all__ = ["KVManager", "HeavyHittersKV", "STACVoxelKV"]
