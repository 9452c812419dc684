"""ctypes binding of libstac_b200.so.  There is no fallback: if the library is missing or a
call fails, an exception is raised."""

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libstac_b200.so")

c_void_p, c_int, c_i64, c_f32, c_size_t = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                           ctypes.c_float, ctypes.c_size_t)

# name -> (restype, argtypes); must list every function declared in include/stac_b200.h
SIGNATURES = {
    "stac_status_string": (ctypes.c_char_p, [c_int]),
    "stac_abi_version": (c_int, []),
    "stac_attn_workspace_bytes": (c_size_t, [c_int, c_int]),
    "stac_attn_colsum": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_i64, c_i64, c_int, c_void_p, c_void_p,
                                 c_i64, c_i64, c_int, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p, c_i64,
                                 c_int, c_int, c_int, c_f32, c_f32, c_void_p, c_size_t, c_void_p, c_void_p]),
    "stac_selftest_bounded_wait": (c_int, [c_int, c_void_p, c_void_p]),
}

_lib = None


class StacError(RuntimeError):
    pass


def lib():
    """Load the shared library once; raise if it is absent (the product has no CPU path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise StacError(f"{LIB_PATH} not found: build it with `python -m stac_b200.build`")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status, what):
    if status != 0:
        msg = lib().stac_status_string(status).decode()
        raise StacError(f"{what} failed: {msg} (status {status})")


def ptr(t):
    """Device pointer of a torch tensor (or None -> NULL)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)
