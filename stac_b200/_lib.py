"""ctypes binding of libstac_b200.so.  There is no fallback: if the library is missing or a
call fails, an exception is raised."""

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libstac_b200.so")

c_void_p, c_int, c_i64, c_f32, c_size_t = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                           ctypes.c_float, ctypes.c_size_t)



class StacPool(ctypes.Structure):
    """Mirror of `struct stac_pool` (include/stac_b200.h)."""
    _fields_ = [
        ("heads", c_int), ("head_dim", c_int), ("elem_bytes", c_int),
        ("pivot_cap", c_int), ("budget_cap", c_int),
        ("voxel_cap", c_int), ("voxel_used", c_int),
        ("sim_thresh", c_f32), ("replace_thresh", c_f32), ("score_thresh", c_f32),
        ("buf_K", c_void_p), ("buf_V", c_void_p), ("buf_S", c_void_p),
        ("buf_row_seg", c_void_p), ("buf_row_cnt", c_void_p), ("buf_free", c_void_p), ("buf_cap", c_int),
        ("piv_K", c_void_p), ("piv_V", c_void_p), ("piv_W", c_void_p), ("piv_S", c_void_p), ("piv_C", c_void_p),
        ("piv_row_seg", c_void_p), ("piv_row_cnt", c_void_p), ("piv_cap", c_int),
        ("over_K_in", c_void_p), ("over_V_in", c_void_p), ("over_S_in", c_void_p),
        ("over_hv_in", c_void_p), ("over_start_in", c_void_p),
        ("over_K_out", c_void_p), ("over_V_out", c_void_p), ("over_S_out", c_void_p),
        ("over_hv_out", c_void_p), ("over_start_out", c_void_p),
        ("over_cap", c_int),
        ("meta", c_void_p),
        ("voxel_count", c_void_p),
    ]


class StacEvicted(ctypes.Structure):
    """Mirror of `struct stac_evicted` (include/stac_b200.h)."""
    _fields_ = [
        ("k", c_void_p), ("v", c_void_p),
        ("kv_head_stride", c_i64), ("kv_row_stride", c_i64),
        ("scores", c_void_p), ("voxel_ids", c_void_p),
        ("meta_head_stride", c_i64),
        ("positions", c_void_p),
        ("tokens_per_head", c_int),
    ]


(META_BUF_TOP, META_BUF_FREE_LEN, META_PIV_TOP, META_OVER_COUNT, META_BUF_USED, META_PIV_USED, META_DROPPED,
 META_VOXELS) = range(8)
META_SIZE = 8
VOXEL_MAX_POINTS = 131072

# name -> (restype, argtypes); must list every function declared in include/stac_b200.h
SIGNATURES = {
    "stac_status_string": (ctypes.c_char_p, [c_int]),
    "stac_abi_version": (c_int, []),
    "stac_attn_workspace_bytes": (c_size_t, [c_int, c_int]),
    "stac_attn_colsum": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_i64, c_i64, c_int, c_void_p, c_void_p,
                                 c_i64, c_i64, c_int, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p, c_i64,
                                 c_int, c_int, c_int, c_f32, c_f32, c_void_p, c_size_t, c_void_p, c_void_p]),
    "stac_attn_colsum_noalloc": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_i64, c_i64, c_int, c_void_p,
                                         c_void_p, c_i64, c_i64, c_int, c_void_p, c_i64, c_void_p, c_i64, c_void_p,
                                         c_void_p, c_i64, c_int, c_int, c_int, c_f32, c_f32, c_void_p, c_void_p]),
    "stac_selftest_bounded_wait": (c_int, [c_int, c_void_p, c_void_p]),
    "stac_voxel_scratch_bytes": (c_size_t, [c_int]),
    "stac_voxel_hash_clear": (c_int, [c_void_p, c_i64, c_void_p]),
    "stac_voxel_rehash": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_i64, c_void_p]),
    "stac_voxel_upsert": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_f32, c_void_p, c_int, c_void_p, c_void_p, c_i64,
                                  c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "stac_pointmap_to_positions": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_f32, c_void_p,
                                           c_void_p, c_void_p]),
    "stac_voxel_neighbors": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_i64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "stac_append_kv": (c_int, [c_void_p, c_void_p, c_i64, c_i64, c_i64, c_i64, c_void_p, c_void_p, c_i64, c_void_p,
                               c_i64, c_int, c_int, c_int, c_i64, c_int, c_int, c_void_p]),
    "stac_qkv_epilogue_append": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_void_p, c_void_p, c_f32, c_void_p,
                                         c_void_p, c_void_p, c_int, c_void_p, c_i64, c_void_p, c_void_p, c_i64,
                                         c_void_p, c_i64, c_int, c_int, c_int, c_i64, c_void_p]),
    "stac_scores_update": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_i64, c_int, c_int, c_int, c_int, c_f32,
                                   c_void_p]),
    "stac_h2o_select": (c_int, [c_void_p, c_i64, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "stac_compact": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p]),
    "stac_merge_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "stac_merge_insert": (c_int, [ctypes.POINTER(StacPool), ctypes.POINTER(StacEvicted), c_void_p, c_size_t, c_int,
                                  c_void_p, c_void_p]),
    "stac_retrieve": (c_int, [ctypes.POINTER(StacPool), c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p]),
}

# kernels launched by one call of each entry point (the upper figure where it depends on arguments);
# used to report how many of this library's kernels ran in a timed region
# (stac_attn_colsum: fast forward, exact forward, column sums)
KERNELS_PER_CALL = {
    "stac_attn_colsum": 3, "stac_attn_colsum_noalloc": 3, "stac_selftest_bounded_wait": 1,
    "stac_voxel_hash_clear": 1, "stac_voxel_rehash": 2, "stac_voxel_upsert": 3, "stac_voxel_neighbors": 2, "stac_pointmap_to_positions": 1,
    "stac_append_kv": 1, "stac_qkv_epilogue_append": 1, "stac_scores_update": 1, "stac_h2o_select": 1, "stac_compact": 2, "stac_merge_insert": 16, "stac_retrieve": 2,
}
CALLS = {}


class _CountingLib:
    """Forwards to the ctypes handle and counts calls per entry point."""

    def __init__(self, handle):
        self._handle = handle

    def __getattr__(self, name):
        fn = getattr(self._handle, name)
        if name not in KERNELS_PER_CALL:
            return fn

        def counted(*args):
            CALLS[name] = CALLS.get(name, 0) + 1
            return fn(*args)
        self.__dict__[name] = counted
        return counted


def kernel_launches():
    """Kernels of this library launched so far (by the entry-point calls made through lib())."""
    return sum(KERNELS_PER_CALL[n] * c for n, c in CALLS.items())


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
        _lib = _CountingLib(handle)
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
