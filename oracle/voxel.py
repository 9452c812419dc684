"""Oracle for the point -> voxel-id table (test infrastructure).

Restates stac/stac_voxel.py:339-340 (quantisation), stac/voxel.py:60-71 (key packing),
stac/voxel.py:195-324 (append-only upsert with stable ids) and stac/voxel.py:371-521
together with stac/stac_voxel.py:294-323 (Chebyshev-cube neighbour lookup).
"""

import numpy as np

from .numerics import f32

KEY_BIAS = 1 << 20
KEY_SHIFT_Y = 21
KEY_SHIFT_Z = 42


def quantize(points, voxel_size):
    """ijk = floor(points / voxel_size) in float32 with true division, cast to int32."""
    p = f32(points)
    vs = np.float32(voxel_size)
    return np.floor(p / vs).astype(np.int32)


def pack_keys(ijk):
    """key = (i+2^20) + (j+2^20)*2^21 + (k+2^20)*2^42 as int64."""
    a = np.asarray(ijk).astype(np.int64) + KEY_BIAS
    return a[:, 0] + (a[:, 1] << KEY_SHIFT_Y) + (a[:, 2] << KEY_SHIFT_Z)


def neighbor_offsets(R):
    """Packed additive key offsets of the (2R+1)^3 cube, in (dx, dy, dz) lexicographic order."""
    r = np.arange(-R, R + 1, dtype=np.int64)
    dx, dy, dz = np.meshgrid(r, r, r, indexing="ij")
    return (dx + (dy << KEY_SHIFT_Y) + (dz << KEY_SHIFT_Z)).reshape(-1)


class VoxelTable:
    """Append-only table: id = row number; keys never move once inserted."""

    def __init__(self, voxel_size=0.05):
        self.voxel_size = np.float32(voxel_size)
        self.keys = np.empty(0, np.int64)      # packed key of voxel id i
        self.ijk = np.empty((0, 3), np.int32)  # integer coordinates of voxel id i

    @property
    def num_voxels(self):
        return int(self.keys.shape[0])

    def lookup(self, keys):
        """ids of packed keys, -1 where absent."""
        keys = np.asarray(keys, np.int64)
        out = np.full(keys.shape, -1, np.int32)
        if self.keys.size == 0 or keys.size == 0:
            return out
        order = np.argsort(self.keys, kind="stable")
        sk = self.keys[order]
        pos = np.clip(np.searchsorted(sk, keys), 0, sk.size - 1)
        hit = sk[pos] == keys
        out[hit] = order[pos[hit]].astype(np.int32)
        return out

    def upsert(self, ijk):
        """Insert integer coordinates [n,3]; return their stable ids [n] int32.

        Known keys keep their id.  Keys new in this call are ranked among themselves in
        ascending packed-key order and get ids n_old + rank.
        """
        ijk = np.asarray(ijk, np.int32).reshape(-1, 3)
        if ijk.shape[0] == 0:
            return np.empty(0, np.int32)
        keys = pack_keys(ijk)
        ids = self.lookup(keys)
        new = ids < 0
        if new.any():
            uniq, first, inv = np.unique(keys[new], return_index=True, return_inverse=True)
            base = self.num_voxels
            ids[new] = (base + inv).astype(np.int32)
            self.keys = np.concatenate([self.keys, uniq])
            self.ijk = np.concatenate([self.ijk, ijk[new][first]])
        return ids

    def neighbors(self, voxel_ids, R=2):
        """Sorted unique ids of existing voxels in the Chebyshev cube of radius R around
        each queried id (self included)."""
        q = np.asarray(voxel_ids, np.int64).reshape(-1)
        q = q[(q >= 0) & (q < self.num_voxels)]
        if q.size == 0:
            return np.empty(0, np.int64)
        cand = (self.keys[q][:, None] + neighbor_offsets(R)[None, :]).reshape(-1)
        ids = self.lookup(cand)
        return np.unique(ids[ids >= 0]).astype(np.int64)


def recent_neighbor_ids(table, token_voxel_ids, recent_tokens, seen_ids, R=2):
    """Voxel set queried at retrieval (stac/stac_voxel.py:294-323).

    token_voxel_ids: voxel id per live hot-cache position (head 0 of the last layer slot).
    If fewer than ``recent_tokens`` positions are live, every voxel id seen so far is
    returned (in the order given by ``seen_ids``); otherwise the neighbours of the unique
    non-negative ids of the last ``recent_tokens`` positions.
    """
    t = np.asarray(token_voxel_ids)
    if t.size == 0:
        return None
    if t.size < recent_tokens:
        return np.asarray(list(seen_ids), np.int64)
    last = t[t.size - recent_tokens:]
    last = np.unique(last[last >= 0])
    return table.neighbors(last, R)
