"""stac_b200: B200 (sm_100a) implementation of STAC's KV-cache compression hot path behind
the reference's `stac/` operator API.  Host side is Python/PyTorch (tensors, streams); all
compute is hand-written CUDA in libstac_b200.so, reached through a C ABI (include/stac_b200.h).
"""

__version__ = "0.1.0"
