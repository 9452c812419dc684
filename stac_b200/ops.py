"""Thin torch-tensor wrappers over the C ABI (one function per entry point)."""

import math

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr


class DeviceStatus:
    """One int32 in device memory that kernels set when a bounded wait or capacity check
    fails.  ``raise_if_set`` synchronises and raises; call it where a sync is acceptable."""

    NAMES = {1: "TMA wait timed out", 2: "MMA wait timed out", 3: "consumer wait timed out",
             4: "sort scratch too small", 5: "segment pool exhausted", 6: "self-test timeout"}

    def __init__(self, device):
        self.word = torch.zeros(1, dtype=torch.int32, device=device)

    def read(self):
        return int(self.word.item())

    def clear(self):
        self.word.zero_()

    def raise_if_set(self, what="kernel"):
        code = self.read()
        if code != 0:
            self.clear()
            raise _lib.StacError(f"{what}: device error {code} ({self.NAMES.get(code, 'unknown')})")


class LaggedInts:
    """Device int32 values mirrored on the host WITHOUT a synchronisation at the producing call:
    ``push`` enqueues copies into pinned host memory on the current stream and records an event;
    ``pull`` is made by the NEXT call that needs the numbers, by which time that event lies a
    whole stream step in the past, so waiting for it does not stall a host that runs at most
    one step ahead of the GPU.  ``pull`` returns None when nothing is pending."""

    def __init__(self, n):
        self.pin = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.event = None

    def push(self, *tensors):
        off = 0
        for t in tensors:
            n = t.numel()
            self.pin[off:off + n].copy_(t.reshape(-1), non_blocking=True)
            off += n
        self.event = torch.cuda.Event()
        self.event.record()

    def pending(self):
        return self.event is not None

    def pull(self):
        if self.event is None:
            return None
        self.event.synchronize()
        self.event = None
        return self.pin.tolist()


_workspaces = {}


def _attn_workspace(device, M, H):
    """Scratch of stac_attn_colsum (row log-sum-exps, split partials, arrival counters).  One per
    (device, stream): calls on one stream are ordered and may share it, calls issued on different
    streams may overlap on the GPU and must not."""
    need = _lib.lib().stac_attn_workspace_bytes(M, H)
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() * 4 < need:
        ws = torch.empty(max(need // 4, 1), dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def _kv_strides(t, layout):
    """(row_stride, head_stride) in elements for a [H,T,D] ('htd') or [T,H,D] ('thd') tensor."""
    assert t.stride(-1) == 1
    if layout == "htd":
        return t.stride(1), t.stride(0)
    return t.stride(0), t.stride(1)


def attn_colsum(q, k_hot, v_hot, T_hot, k_ret=None, v_ret=None, bias_ret=None, T_ret=0, *,
                layout="htd", scale=None, subsample_ratio=1.0, want_lse=False, want_colsum=True,
                out=None, colsum=None, status=None):
    """q [M,H,64] bf16 (row stride arbitrary); hot and retrieved keys/values in ``layout``;
    bias_ret [H, >=T_ret] fp32.  Returns (out [M,H,64] bf16, lse [H,M] | None,
    colsum [H, T_hot+T_ret] fp32 | None)."""
    assert q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 3 and q.stride(2) == 1
    M, H, D = q.shape
    assert q.stride(1) == D, "heads of a query row must be contiguous"
    dev = q.device
    if out is None:
        out = torch.empty((M, H, D), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((H, M), dtype=torch.float32, device=dev) if want_lse else None
    N = T_hot + T_ret
    if want_colsum and colsum is None:
        colsum = torch.empty((H, N), dtype=torch.float32, device=dev)
    if not want_colsum:
        colsum = None
    ws = _attn_workspace(dev, M, H)
    hr, hh = _kv_strides(k_hot, layout) if T_hot > 0 else (D, D)
    if T_hot > 0:
        assert _kv_strides(v_hot, layout) == (hr, hh)
    rr, rh = (D, D)
    if T_ret > 0:
        rr, rh = _kv_strides(k_ret, layout)
        assert _kv_strides(v_ret, layout) == (rr, rh)
        assert bias_ret.dtype == torch.float32 and bias_ret.stride(1) == 1
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    st = _lib.lib().stac_attn_colsum(
        ptr(q), q.stride(0),
        ptr(k_hot) if T_hot > 0 else None, ptr(v_hot) if T_hot > 0 else None, hr, hh, T_hot,
        ptr(k_ret) if T_ret > 0 else None, ptr(v_ret) if T_ret > 0 else None, rr, rh, T_ret,
        ptr(bias_ret) if T_ret > 0 else None, bias_ret.stride(0) if T_ret > 0 else 0,
        ptr(out), out.stride(0), ptr(lse), ptr(colsum), colsum.stride(0) if colsum is not None else 0,
        M, H, D, float(scale), float(subsample_ratio), ptr(ws), ws.numel() * 4,
        ptr(status.word) if status is not None else None, stream_ptr())
    check(st, "stac_attn_colsum")
    return out, lse, colsum


def flash_attn_bias_colsum(q, k, v, bias=None, softmax_scale=None, return_colsum=False,
                           subsample_ratio=1.0):
    """Same call as the reference's attn_cuda.flash_attn_bias_colsum
    (attn-cuda/attn_cuda/__init__.py:6-43): q [B,M,H,D], k/v [B,N,H,D] bf16 with B == 1,
    bias [B,H,1,N] or [B,H,N] (per-key).  Returns (out [B,M,H,D], lse [B,H,M][, colsum [B,H,N]])."""
    if q.dim() != 4 or q.shape[0] != 1:
        raise ValueError("batch size 1 only")
    if q.shape[-1] != 64:
        raise ValueError("Only head_dim=64 is supported")
    if not (0.0 < subsample_ratio <= 1.0):
        raise ValueError("subsample_ratio must be in (0, 1]")
    q3, k3, v3 = q[0].contiguous(), k[0].contiguous(), v[0].contiguous()
    N = k3.shape[0]
    if bias is None:
        o, lse, cs = attn_colsum(q3, k3, v3, N, layout="thd", scale=softmax_scale,
                                 subsample_ratio=subsample_ratio, want_lse=True,
                                 want_colsum=return_colsum)
    else:
        b = bias
        if b.dim() == 4:
            if b.shape[2] != 1:
                raise ValueError("4D bias must have shape [B, H, 1, N]")
            b = b.squeeze(2)
        b = b[0].to(torch.float32).contiguous()
        # every key carries a bias: treat all of them as the biased segment
        o, lse, cs = attn_colsum(q3, None, None, 0, k3, v3, b, N, layout="thd", scale=softmax_scale,
                                 subsample_ratio=subsample_ratio, want_lse=True,
                                 want_colsum=return_colsum)
    res = (o.unsqueeze(0), lse.unsqueeze(0))
    if return_colsum:
        res = res + (cs.unsqueeze(0),)
    return res
