"""Point maps -> one world point per token, the input of ``STACVoxelKV.append_positions``.

``pointmap_to_positions`` does what ``StreamSession.get_pointmap`` does for the "pointmap"
prediction mode (stream_session.py:213-256): bilinear reduction of the predicted world points and
of their confidence to one sample per patch, `special_tokens_size` zero points in front of every
frame, mask = confidence > threshold -- in one kernel reading the [S,H,W,3] map in place instead of
two permutes, two interpolate calls, a reshape and two concatenations.
"""

from typing import Tuple

import torch

from .. import _lib
from .._lib import check, ptr, stream_ptr


@torch.no_grad()
def pointmap_to_positions(world_points: torch.Tensor, world_points_conf: torch.Tensor, patch_size: int,
                          conf_threshold: float = 1.0, special_tokens_size: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """world_points [B,S,H,W,3] or [S,H,W,3], world_points_conf [B,S,H,W] or [S,H,W] (B == 1), CUDA.
    Returns (pts3d f32 [S, special + H'W', 3], valid_mask bool [S, special + H'W'])."""
    if world_points.dim() == 5:
        assert world_points.shape[0] == 1, "Batch size must be 1."
        world_points, world_points_conf = world_points[0], world_points_conf[0]
    assert world_points.is_cuda, "pointmap_to_positions requires CUDA tensors"
    S, H, W, C = world_points.shape
    assert C == 3 and tuple(world_points_conf.shape) == (S, H, W)
    wp = world_points.to(torch.float32).contiguous()
    cf = world_points_conf.to(torch.float32).contiguous()
    n_tok = special_tokens_size + max(1, H // patch_size) * max(1, W // patch_size)
    pts = torch.empty((S, n_tok, 3), dtype=torch.float32, device=wp.device)
    mask = torch.empty((S, n_tok), dtype=torch.bool, device=wp.device)
    check(_lib.lib().stac_pointmap_to_positions(ptr(wp), ptr(cf), S, H, W, int(patch_size), int(special_tokens_size),
                                                float(conf_threshold), ptr(pts), ptr(mask), stream_ptr()),
          "stac_pointmap_to_positions")
    return pts, mask
