"""GPU voxel table behind the reference's ``BinaryVoxel`` interface (stac/voxel.py:19-566).

Ids are row numbers of an append-only table and are assigned exactly as the reference does
(known keys keep their id; keys new in a call get ``n_old + rank`` among the sorted new unique
keys, stac/voxel.py:256-324).  Membership lives in a device hash table; the sorted key cache,
voxel centres and Morton zones of the reference are not kept (the zones only steer the
reference's CUDA segment allocator and influence no output).
"""

import torch

from .. import _lib
from .._lib import check, ptr, stream_ptr
from ..ops import LaggedInts


def _pow2_at_least(n):
    p = 1
    while p < n:
        p <<= 1
    return p


class BinaryVoxel:
    def __init__(self, voxel_size: float = 0.05, device="cuda", capacity: int = 1 << 15, status=None):
        self._voxel_size = float(voxel_size)
        self.device = torch.device(device)
        self._status = status
        self._init_capacity = int(capacity)
        self._alloc(self._init_capacity)

    def _alloc(self, cap):
        dev = self.device
        self._cap = max(16, (int(cap) + 15) // 16 * 16)   # the flag array is scanned 16 bytes at a time
        self._hash_cap = _pow2_at_least(4 * self._cap)
        self._table_keys = torch.zeros(self._cap, dtype=torch.int64, device=dev)
        self._hash_keys = torch.empty(self._hash_cap, dtype=torch.int64, device=dev)
        self._hash_vals = torch.empty(self._hash_cap, dtype=torch.int32, device=dev)
        self._n_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self._flags = torch.zeros(self._cap, dtype=torch.uint8, device=dev)
        self._nbr_ids = torch.empty(self._cap, dtype=torch.int32, device=dev)
        self._nbr_count = torch.zeros(1, dtype=torch.int32, device=dev)
        self._scratch = torch.empty(_lib.lib().stac_voxel_scratch_bytes(_lib.VOXEL_MAX_POINTS),
                                    dtype=torch.uint8, device=dev)
        self._n = 0                 # voxel count as of the last call whose result was read back
        self._unread = 0            # points upserted since then: count <= _n + _unread
        self._mirror = LaggedInts(1)
        check(_lib.lib().stac_voxel_hash_clear(ptr(self._hash_keys), self._hash_cap, stream_ptr()),
              "stac_voxel_hash_clear")

    def reset(self):
        self._alloc(self._init_capacity)

    def _grow(self, need):
        """Make room for `need` voxels: larger key table, flags and a rehash."""
        new_cap = self._cap
        while new_cap < need:
            new_cap *= 2
        self._sync_count()
        old_keys, n_dev, n = self._table_keys, self._n_dev, self._n
        self._alloc(new_cap)
        self._table_keys[: old_keys.numel()].copy_(old_keys)
        self._n_dev.copy_(n_dev)
        self._n = n
        check(_lib.lib().stac_voxel_rehash(ptr(self._table_keys), ptr(self._n_dev), self._cap,
                                           ptr(self._hash_keys), ptr(self._hash_vals), self._hash_cap,
                                           stream_ptr()), "stac_voxel_rehash")

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        """The table is its key list (id = position); the hash table is rebuilt on load."""
        self._sync_count()
        return {"n": int(self._n), "table_keys": self._table_keys[: self._n].cpu()}

    def load_state_dict(self, sd):
        n = int(sd["n"])
        self._alloc(self._init_capacity)
        if n > self._cap:
            self._grow(n)
        self._table_keys[:n].copy_(sd["table_keys"])
        self._n, self._unread = n, 0
        self._n_dev.fill_(n)
        check(_lib.lib().stac_voxel_rehash(ptr(self._table_keys), ptr(self._n_dev), self._cap,
                                           ptr(self._hash_keys), ptr(self._hash_vals), self._hash_cap,
                                           stream_ptr()), "stac_voxel_rehash")

    # ------------------------------------------------------------------ voxel count on the host
    def _pull_count(self):
        """Take in the count that the previous upsert left in pinned memory (its copy was enqueued
        behind that call's kernels, a whole step ago)."""
        vals = self._mirror.pull()
        if vals is not None:
            self._n, self._unread = int(vals[0]), 0

    def _sync_count(self):
        """Exact count now (waits for the last upsert if its result has not been read yet)."""
        self._pull_count()

    def voxel_num_bound(self) -> int:
        """Upper bound of the voxel count that never waits for the GPU: the last count read back
        plus the points upserted since.  Enough to size arrays and to filter ids (ids handed out so
        far are below the true count)."""
        return self._n + self._unread

    # ------------------------------------------------------------------ upsert
    def _upsert(self, points, ijk, mask, n):
        if n == 0:
            return torch.empty(0, dtype=torch.int32, device=self.device)
        if n > _lib.VOXEL_MAX_POINTS:
            raise ValueError(f"at most {_lib.VOXEL_MAX_POINTS} points per upsert call, got {n}")
        self._pull_count()
        if self._n + n > self._cap:
            self._grow(self._n + n)
        ids = torch.empty(n, dtype=torch.int32, device=self.device)
        st = _lib.lib().stac_voxel_upsert(
            ptr(points), ptr(ijk), ptr(mask), n, self._voxel_size, ptr(self._table_keys), self._cap,
            ptr(self._hash_keys), ptr(self._hash_vals), self._hash_cap, ptr(self._n_dev), ptr(ids),
            ptr(self._scratch), self._scratch.numel(),
            ptr(self._status.word) if self._status is not None else None, stream_ptr())
        check(st, "stac_voxel_upsert")
        # the new count travels to pinned memory behind the kernels; nobody waits for it here
        self._unread += n
        self._mirror.push(self._n_dev)
        return ids

    @torch.no_grad()
    def upsert(self, ijk_valid: torch.Tensor) -> torch.Tensor:
        """ijk_valid [N,3] int32 -> stable voxel ids [N] int32 (stac/voxel.py:195-324)."""
        if ijk_valid.numel() == 0:
            return torch.empty(0, dtype=torch.int32, device=self.device)
        assert ijk_valid.shape[-1] == 3, "ijk_valid must be [N,3]"
        ijk = ijk_valid.to(device=self.device, dtype=torch.int32).contiguous()
        return self._upsert(None, ijk, None, ijk.shape[0])

    @torch.no_grad()
    def upsert_points(self, points: torch.Tensor, mask: torch.Tensor = None) -> torch.Tensor:
        """Fused quantise + upsert of world points [N,3] fp32; masked-out points get id -1
        (stac/stac_voxel.py:339-347)."""
        pts = points.to(device=self.device, dtype=torch.float32).contiguous()
        m = None if mask is None else mask.to(device=self.device, dtype=torch.uint8).contiguous()
        return self._upsert(pts, None, m, pts.shape[0])

    # ------------------------------------------------------------------ neighbours
    @torch.no_grad()
    def neighbor_ids(self, token_voxel_ids: torch.Tensor = None, radius_cells: int = 2, all_ids: bool = False):
        """Ascending unique ids of existing voxels within `radius_cells` (Chebyshev) of the given
        voxel ids.  Returns (ids int32 [capacity] view, count int32 [1]) on the device; only the
        first `count` entries are meaningful and both are overwritten by the next call."""
        n_tok = 0 if token_voxel_ids is None else int(token_voxel_ids.numel())
        if token_voxel_ids is not None:
            assert token_voxel_ids.dtype == torch.int32 and token_voxel_ids.is_contiguous()
        st = _lib.lib().stac_voxel_neighbors(
            ptr(token_voxel_ids), n_tok, int(radius_cells), 1 if all_ids else 0, ptr(self._table_keys),
            ptr(self._n_dev), self._cap, ptr(self._hash_keys), ptr(self._hash_vals), self._hash_cap,
            ptr(self._flags), ptr(self._nbr_ids), ptr(self._nbr_count), stream_ptr())
        check(st, "stac_voxel_neighbors")
        return self._nbr_ids, self._nbr_count

    @torch.no_grad()
    def neighbors(self, voxel_ids: torch.Tensor, radius_m: float, include_self: bool = True):
        """Sorted unique neighbour ids (the only part of the reference's (ids, dist2, found)
        result that the managers consume, stac/stac_voxel.py:316-323).  Self is always included."""
        import math
        R = max(1, int(math.ceil(radius_m / self._voxel_size)))
        ids, count = self.neighbor_ids(voxel_ids.to(self.device, torch.int32).contiguous(), R)
        return ids[: int(count.item())].to(torch.int64)

    # ------------------------------------------------------------------ accessors
    def get_voxel_num(self) -> int:
        """Exact number of voxels (waits for the last upsert to finish if need be)."""
        self._sync_count()
        return self._n

    def get_voxel_size(self) -> float:
        return self._voxel_size

    def get_voxel_keys_1d(self) -> torch.Tensor:
        self._sync_count()
        return self._table_keys[: self._n]

    def get_voxel_keys(self) -> torch.Tensor:
        """Integer coordinates [N,3] int32, unpacked from the 63-bit keys."""
        self._sync_count()
        k = self._table_keys[: self._n]
        off = 1 << 20
        m = (1 << 21) - 1
        return torch.stack([(k & m) - off, ((k >> 21) & m) - off, ((k >> 42) & m) - off], 1).to(torch.int32)

    def get_centers(self, voxel_ids: torch.Tensor) -> torch.Tensor:
        return (self.get_voxel_keys()[voxel_ids.long()].to(torch.float32) + 0.5) * self._voxel_size

    def get_voxel_info(self):
        return {"voxel_size": self._voxel_size, "voxel_keys": self.get_voxel_keys(),
                "voxel_keys_1d": self.get_voxel_keys_1d()}
