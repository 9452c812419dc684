"""Oracle for the manager level of the path (test infrastructure): hot cache, H2O scores
and selection, eviction into the voxel memory and pivot retrieval, driven per chunk in the
reference's call order  append_kv (all layers) -> scores -> append_positions -> [retrieve]
-> prune.

Restates stac/kv_manager.py:227-309 (append), stac/h2o.py:177-216 (score update),
stac/h2o.py:244-354 (keep set), stac/h2o.py:356-436 and stac/stac_voxel.py:409-419
(compaction), stac/stac_voxel.py:326-365 (positions), stac/stac_voxel.py:421-488 (eviction)
and stac/stac_voxel.py:665-762 (retrieval hand-off).  Column sums are injected by the
caller, as the attention kernel has its own oracle.
"""

import numpy as np

from .numerics import f32, make_rounder
from .pool import VoxelMerger
from .voxel import VoxelTable, quantize, recent_neighbor_ids


def h2o_keep_indices(scores, T, recent_tokens, pinned_positions, hh_tokens, hot_tokens):
    """Keep set per (layer, head) row of ``scores`` [..., >=T]; returns int64 [..., T'] or
    None when nothing is pruned.  Ties at the k-th score resolve to the lower position."""
    if T <= max(hot_tokens, recent_tokens):
        return None
    recent_keep = min(recent_tokens, T)
    base = np.arange(T - recent_keep, T, dtype=np.int64)
    pinned = np.asarray(pinned_positions, np.int64)
    pinned = pinned[(pinned >= 0) & (pinned < T)]
    if pinned.size:
        base = np.unique(np.concatenate([pinned, base]))
    if base.size == T:
        return None
    mask = np.ones(T, bool)
    mask[base] = False
    prefix = np.nonzero(mask)[0]
    lead = scores.shape[:-1]
    k = min(hh_tokens, prefix.size)
    if k == 0:
        return np.broadcast_to(base, lead + (base.size,)).copy()
    if k == prefix.size:
        keep = np.sort(np.concatenate([base, prefix]))
        return np.broadcast_to(keep, lead + (keep.size,)).copy()
    sp = f32(scores[..., :T])[..., prefix]
    order = np.argsort(-sp, axis=-1, kind="stable")[..., :k]
    hh = prefix[order]
    base_b = np.broadcast_to(base, lead + (base.size,))
    return np.sort(np.concatenate([base_b, hh], axis=-1), axis=-1)


class StacManager:
    """Numpy twin of STACVoxelKV with all layers registered and voxelised."""

    def __init__(self, num_layers, num_heads, head_dim, token_per_frame, buffer_size,
                 chunk_size=1, recent_size=1, pinned_idx=(0,), hh_size=0, temperature=1.0,
                 voxel_size=0.05, init_voxels=1024, voxel_buf_cap=8, voxel_piv_cap=4,
                 sim_threshold=0.8, replace_threshold=0.8, score_threshold=0.2,
                 retrieval_size=-1, dtype="f32"):
        self.L, self.H, self.D = num_layers, num_heads, head_dim
        self.tpf = token_per_frame
        self.temperature = np.float32(temperature)
        pinned = [i for i in pinned_idx if i >= 0]
        hot_frames = hh_size + recent_size + len(pinned)
        if buffer_size <= hot_frames:
            buffer_size = hot_frames + 1
        self.T_buf = buffer_size * token_per_frame
        self.recent_tokens = recent_size * token_per_frame
        self.hh_tokens = hh_size * token_per_frame
        self.hot_tokens = hot_frames * token_per_frame
        self.pinned_positions = np.concatenate(
            [np.arange(i * token_per_frame, (i + 1) * token_per_frame) for i in pinned]
        ) if pinned else np.empty(0, np.int64)
        self.retrieval_tokens = int(retrieval_size * token_per_frame)
        self.rnd = make_rounder(dtype)
        L, H, T, D = self.L, self.H, self.T_buf, self.D
        self.K = np.zeros((L, H, T, D), np.float32)
        self.V = np.zeros((L, H, T, D), np.float32)
        self.TI = np.full((L, H, T), -1, np.int64)
        self.S = np.zeros((L, H, T), np.float32)
        self.SC = np.zeros((L, H, T), np.float32)
        self.VX = np.full((L, H, T), -1, np.int32)
        self.off = [0] * L
        self.off_vx = 0
        self.last_score = [0] * L
        self.frames = 0
        self.table = VoxelTable(voxel_size)
        self.seen = set()
        self.recent_ids = None
        self.merger = VoxelMerger(L * H, D, init_voxels, voxel_piv_cap, voxel_buf_cap,
                                  sim_threshold, replace_threshold, score_threshold, dtype)
        self.ret = None  # (K [L*H,R,D], V, bias [L*H,R]) after a retrieval
        self.last_keep = None

    def append_kv(self, k, v, slot):
        """k, v [H, T_new, D]."""
        t0, n = self.off[slot], k.shape[1]
        assert n % self.tpf == 0 and t0 + n <= self.T_buf
        self.K[slot, :, t0:t0 + n] = self.rnd(k)
        self.V[slot, :, t0:t0 + n] = self.rnd(v)
        f = n // self.tpf
        ids = (np.arange(self.frames, self.frames + f)[:, None] * self.tpf
               + np.arange(self.tpf)[None, :]).reshape(-1)
        self.TI[slot, :, t0:t0 + n] = ids[None, :]
        self.off[slot] = t0 + n
        if slot == self.L - 1:
            self.frames += f

    def update_scores(self, colsum, slot, Tq):
        """colsum [H, T_live] = per-key column sums over the Tq query rows of this step."""
        s = f32(colsum)
        T_live = s.shape[1]
        s = s * np.float32(T_live) / np.float32(Tq)
        old = self.last_score[slot]
        if T_live > old:
            self.S[slot, :, old:T_live] = s[:, old:T_live]
        if old > 0:
            self.S[slot, :, :old] = self.S[slot, :, :old] * self.temperature + s[:, :old]
        self.SC[slot, :, :T_live] += np.float32(1)
        self.last_score[slot] = T_live

    def append_positions(self, points, mask):
        n = points.shape[0]
        if n == 0:
            return
        ijk = quantize(points, self.table.voxel_size)
        valid = np.asarray(mask, bool)
        ids = np.full(n, -1, np.int32)
        if valid.any():
            got = self.table.upsert(ijk[valid])
            ids[valid] = got
            self.seen.update(int(i) for i in got)
        t0 = self.off_vx
        assert all(o == t0 + n for o in self.off)
        self.VX[:, :, t0:t0 + n] = ids[None, None, :]
        self.off_vx = t0 + n
        self.recent_ids = recent_neighbor_ids(
            self.table, self.VX[self.L - 1, 0, : self.off_vx], self.recent_tokens, self.seen, R=2)

    def retrieve(self, return_buf=False):
        if not self.seen or self.recent_ids is None:
            return
        K, V, M, B, idx = self.merger.retrieve(self.recent_ids, self.retrieval_tokens, return_buf)
        Tm = K.shape[1]
        if self.retrieval_tokens >= 0:
            Tm = min(Tm, self.retrieval_tokens)
        self.ret = (K[:, :Tm], V[:, :Tm], B[:, :Tm], M[:, :Tm], idx[:, :Tm])

    def prune(self):
        T = self.off[0]
        assert all(o == T for o in self.off)
        keep = h2o_keep_indices(self.S, T, self.recent_tokens, self.pinned_positions,
                                self.hh_tokens, self.hot_tokens)
        self.last_keep = keep
        if keep is None:
            return
        L, H, D = self.L, self.H, self.D
        Tp = keep.shape[-1]
        drop_mask = np.ones((L, H, T), bool)
        np.put_along_axis(drop_mask, keep, False, axis=2)
        Td = T - Tp
        if Td > 0:
            sel = np.nonzero(drop_mask.reshape(L * H, T))[1].reshape(L * H, Td)
            Kd = np.take_along_axis(self.K[:, :, :T].reshape(L * H, T, D), sel[:, :, None], 1)
            Vd = np.take_along_axis(self.V[:, :, :T].reshape(L * H, T, D), sel[:, :, None], 1)
            Sd = np.take_along_axis(self.S[:, :, :T].reshape(L * H, T), sel, 1)
            VXd = np.take_along_axis(self.VX[:, :, :T].reshape(L * H, T), sel, 1)
            self.merger.insert_and_merge(Kd, Vd, Sd, VXd, self.table.num_voxels)
        for arr, fill in ((self.K, None), (self.V, None), (self.TI, -1), (self.S, 0), (self.SC, 0),
                          (self.VX, -1)):
            if arr.ndim == 4:
                arr[:, :, :Tp] = np.take_along_axis(arr[:, :, :T], keep[..., None], 2)
            else:
                arr[:, :, :Tp] = np.take_along_axis(arr[:, :, :T], keep, 2)
                arr[:, :, Tp:] = fill
        self.off = [Tp] * L
        self.off_vx = Tp
        self.last_score = [min(x, Tp) for x in self.last_score]
