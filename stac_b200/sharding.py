"""Head sharding of one stream across the GPUs of a box.

Every step of the path is independent per (layer, head): attention, scores, H2O selection,
compaction, the voxel-memory rows (row = (layer*H + head, voxel)) and retrieval never mix heads
(stac/merger.py:1211-1214).  A rank therefore runs an ordinary ``STACVoxelKV`` over its slice of
the heads; the voxel table is replicated (every rank sees the same points and assigns the same
ids).  The only exchange is an all-gather of the per-head counts of valid retrieved pivots, so
that every rank knows the retrieval state of all heads (statistics, early-out when no head
retrieved anything).  No K/V crosses NVLink.
"""

import torch
import torch.distributed as dist


def head_slice(rank: int, world: int, num_heads: int) -> slice:
    """Contiguous block of heads owned by `rank`; `world` must divide `num_heads`."""
    if num_heads % world != 0:
        raise ValueError(f"{world} ranks do not divide {num_heads} heads")
    per = num_heads // world
    return slice(rank * per, (rank + 1) * per)


def gather_head_counts(local_counts: torch.Tensor, num_layers: int, group=None) -> torch.Tensor:
    """local_counts int32 [L * H_local] (pool-head order: layer-major) -> int32 [L, H] for all
    heads of the stream, identical on every rank.  One all-gather (NCCL on GPUs, gloo on CPU)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    local = local_counts.reshape(num_layers, -1).to(torch.int32).contiguous()
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local, group=group)
    return torch.cat(parts, dim=1)
