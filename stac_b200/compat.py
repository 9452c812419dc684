"""Make ``import stac`` resolve to this package's drop-in classes.

The reference's callers bind the managers by module path: ``from stac.h2o import
HeavyHittersKV`` (causalvggt/layers/attention.py:19, causalvggt/models/aggregator.py:22) and
``from stac.kv_manager import KVManager`` / ``from stac.stac_voxel import STACVoxelKV``
(stream_session.py:3-4).  ``install_as_stac()`` registers ``stac_b200.stac`` and its
submodules under those names in ``sys.modules``; called before the first import of the
reference's ``causalvggt`` / ``stream_session`` modules it lets ``StreamSession.pipeline`` run
unchanged on this library.
"""

import importlib
import sys

_SUBMODULES = ("kv_manager", "h2o", "stac_voxel", "merger", "voxel")


def install_as_stac():
    """Register the aliases; raises if a different ``stac`` package is already imported."""
    from . import stac as pkg
    have = sys.modules.get("stac")
    if have is not None and have is not pkg:
        raise ImportError(f"another 'stac' package is already imported from {getattr(have, '__file__', '?')}")
    sys.modules["stac"] = pkg
    for name in _SUBMODULES:
        sys.modules["stac." + name] = importlib.import_module("stac_b200.stac." + name)
    return pkg


def uninstall():
    """Remove the aliases (the ``stac_b200.stac`` modules themselves stay imported)."""
    from . import stac as pkg
    if sys.modules.get("stac") is pkg:
        del sys.modules["stac"]
        for name in _SUBMODULES:
            sys.modules.pop("stac." + name, None)
