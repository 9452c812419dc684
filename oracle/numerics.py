"""Number-format helpers shared by the oracle modules (test infrastructure)."""

import numpy as np


def f32(x):
    """Contiguous float32 view/copy of ``x``."""
    a = np.asarray(x, dtype=np.float32)
    return a if a.ndim == 0 else np.ascontiguousarray(a)


def bf16_round(x):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32.

    The pool stores K/V in the cache dtype; with a bf16 cache the reference rounds on
    every write into the pool (``pool[...] = src.to(pool.dtype)``, stac/allocator.py:2861-2866).
    """
    a = f32(x)
    u = a.reshape(-1).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16) << 16
    out = (r & 0xFFFFFFFF).astype(np.uint32).view(np.float32)
    nan = np.isnan(a)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out.reshape(a.shape)


def make_rounder(dtype_name):
    """Return the storage-rounding function for a pool dtype name ('f32' or 'bf16')."""
    if dtype_name == "f32":
        return f32
    if dtype_name == "bf16":
        return bf16_round
    raise ValueError(f"unknown pool dtype {dtype_name!r}")
