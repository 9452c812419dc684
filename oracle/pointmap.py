"""CPU restatement of StreamSession.get_pointmap (stream_session.py:213-256), test infrastructure
only: world points [S,H,W,3] and their confidence [S,H,W] are reduced to one point per patch by
bilinear interpolation (align_corners=False, no antialiasing: the rule of
torch.nn.functional.interpolate), `special` zero points with mask False are put in front of every
frame, and mask = confidence > threshold.

Bilinear rule in fp32, per output index d along an axis of n_in -> n_out samples:
    scale = n_in / n_out;  src = max(scale * (d + 0.5) - 0.5, 0);  i0 = min(int(src), n_in - 1)
    i1 = i0 + (1 if i0 < n_in - 1 else 0);  l1 = clamp(src - i0, 0, 1);  l0 = 1 - l1
The reference hands interpolate a channels-last view ([S,H,W,3] permuted), for which torch's CPU
kernel multiplies the two axis weights first and adds the four taps left to right:
    out = ((h0*w0) * v[i0h,i0w] + (h0*w1) * v[i0h,i1w]) + (h1*w0) * v[i1h,i0w]) + (h1*w1) * v[i1h,i1w]
with every product and sum rounded to fp32.  At 518 x 392 with 14-pixel patches every weight is
exactly 1/4 and this is bit-identical to the reference run on CPU (pinned by
tests/golden/pointmap.npz); at sizes that are not multiples of the patch torch mixes fused and
unfused multiply-adds and agreement is to one unit in the last place.
"""

import numpy as np

from .numerics import f32


def axis_plan(n_in, n_out):
    d = np.arange(n_out, dtype=np.float32)
    scale = np.float32(n_in) / np.float32(n_out)
    src = scale * (d + np.float32(0.5)) - np.float32(0.5)
    src = np.maximum(src, np.float32(0.0)).astype(np.float32)
    i0 = np.minimum(src.astype(np.int64), n_in - 1)
    i1 = i0 + (i0 < n_in - 1)
    l1 = np.clip(src - i0.astype(np.float32), np.float32(0), np.float32(1)).astype(np.float32)
    l0 = (np.float32(1.0) - l1).astype(np.float32)
    return i0, i1, l0, l1


def downsample(x, out_h, out_w):
    """x f32 [S, H, W, C] -> [S, out_h, out_w, C]."""
    x = f32(x)
    H, W = x.shape[1:3]
    h0, h1, a0, a1 = axis_plan(H, out_h)
    w0, w1, b0, b1 = axis_plan(W, out_w)
    taps = ((h0, w0, a0, b0), (h0, w1, a0, b1), (h1, w0, a1, b0), (h1, w1, a1, b1))
    out = None
    for hi, wi, a, b in taps:
        wgt = (a[:, None] * b[None, :]).astype(np.float32)[None, :, :, None]
        term = (wgt * x[:, hi[:, None], wi[None, :]]).astype(np.float32)
        out = term if out is None else (out + term).astype(np.float32)
    return out


def pointmap_to_positions(world_points, conf, patch, conf_threshold, special):
    """world_points f32 [S,H,W,3], conf f32 [S,H,W] -> (pts f32 [S, special + H'W', 3], mask bool)."""
    wp, cf = f32(world_points), f32(conf)
    S, H, W, C = wp.shape
    oh, ow = max(1, H // patch), max(1, W // patch)
    p = downsample(wp, oh, ow)                                    # [S, oh, ow, 3]
    c = downsample(cf[..., None], oh, ow)[..., 0]                 # [S, oh, ow]
    pts = np.concatenate([np.zeros((S, special, C), np.float32), p.reshape(S, oh * ow, C)], axis=1)
    mask = np.concatenate([np.zeros((S, special), bool), c.reshape(S, oh * ow) > np.float32(conf_threshold)], axis=1)
    return pts, mask
