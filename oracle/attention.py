"""fp32 oracle for window+pivot attention with per-key softmax column sums.

Test infrastructure.  Follows the reference's own fp32 check
(stac/flash_attn_triton.py:1018-1036: scores = q k^T * scale + bias, lse = logsumexp,
P = softmax, colsum = P.sum over query rows, O = P v) and its row sub-sampling rule
(attn-cuda/csrc/bindings.cpp:63-83; stac/flash_attn_triton.py:964-974 and :1003-1004).
"""

import math

import numpy as np

from .numerics import f32


def subsample_plan(M, ratio, block_m=128, rule="cuda"):
    """Return (M_sub, row_stride, correction) for the column-sum pass.

    rule="cuda" is the reference's default backend (attn-cuda/csrc/bindings.cpp:63-83) and what
    the library implements; rule="triton" is the Triton entry point
    (stac/flash_attn_triton.py:964-974), used only to compare this oracle with fixtures made by
    running that entry point.

    ratio >= 0.999999 is exact over all M rows (attn-cuda/csrc/bindings.cpp:67-71, the
    default backend; the Triton entry point lacks this special case and drops the last
    M % 128 rows even at ratio 1).  Otherwise M_sub = max(block_m, int(M*ratio)) rounded
    down to a multiple of block_m; if that covers all rows the pass is exact, else rows
    0, s, 2s, ... (s = M // M_sub) are used and the sums are scaled by M / M_sub.
    """
    if ratio >= 0.999999 and rule == "cuda":
        return M, 1, 1.0
    m_sub = max(block_m, int(M * ratio))
    m_sub = (m_sub // block_m) * block_m
    if m_sub >= M:
        return M, 1, 1.0
    return m_sub, max(1, M // m_sub), M / m_sub


def attn_colsum(q, k, v, bias=None, scale=None, subsample_ratio=1.0, rule="cuda"):
    """q [M,H,D], k/v [N,H,D] (token-major, like the reference's [B,T,H,D] with B=1),
    bias [H,N] float32 or None.  Returns O [M,H,D], lse [H,M], colsum [H,N] (float32)."""
    q = f32(q)
    k = f32(k)
    v = f32(v)
    M, H, D = q.shape
    N = k.shape[0]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    out = np.empty((M, H, D), np.float32)
    lse = np.empty((H, M), np.float32)
    colsum = np.empty((H, N), np.float32)
    m_sub, stride, corr = subsample_plan(M, subsample_ratio, rule=rule)
    rows = np.arange(m_sub) * stride
    for h in range(H):
        s = (q[:, h, :] @ k[:, h, :].T) * np.float32(scale)
        if bias is not None:
            s = s + f32(bias[h])[None, :]
        mx = np.max(s, axis=1, keepdims=True)
        mx = np.where(np.isfinite(mx), mx, 0.0).astype(np.float32)
        e = np.exp(s - mx)
        l = e.sum(axis=1, keepdims=True)
        p = e / l
        lse[h] = (mx + np.log(l))[:, 0]
        out[:, h, :] = p @ v[:, h, :]
        colsum[h] = p[rows].sum(axis=0) * np.float32(corr)
    return out, lse, colsum
