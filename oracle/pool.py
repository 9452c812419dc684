"""Oracle for the voxel memory: segment pools, eviction merge and pivot retrieval.

Test infrastructure.  Restates the reference's Python path with the production
allocator (``allocator="segment"``, ``seg_size=1``):

* row -> segment map, LIFO free list and bump allocation:
  stac/allocator.py:2237-2263 (alloc), :2266-2271 (free), :2306-2319 (clean_rows),
  :2321-2345 (segments handed out in ascending row, ascending column order)
* Top-B append with overflow: stac/allocator.py:559-723
* one call of insert_and_merge: stac/merger.py:1157-1255 (filter, row = head*V_alloc+voxel,
  stable sort) and :765-918 (order of operations)
* token -> existing pivot merge: stac/merger.py:586-760
* full buffer -> one pivot: stac/merger.py:408-461
* pivot insert / victim re-merge: stac/merger.py:462-582
* retrieval: stac/merger.py:1377-1543

Rows are addressed as (head, voxel) here; the reference's flattened row number
``head * V_alloc + voxel`` only fixes the processing order, which is (head, voxel) ascending.
Everything is float32 except where the reference computes in the pool dtype.
"""

import math

import numpy as np

from .numerics import bf16_round, f32, make_rounder

RESERVED, AVAILABLE, FULL = 0, 1, 2


class SegmentPool:
    """One token per segment.  ``row_seg[h, v, c]`` is the segment holding column c of row
    (h, v), or -1; ``row_offset`` the number of occupied columns; ``row_state`` the row FSM."""

    def __init__(self, heads, cap, fields):
        self.H = heads
        self.cap = cap
        self.V = 0
        self.row_state = np.zeros((heads, 0), np.int8)
        self.row_offset = np.zeros((heads, 0), np.int32)
        self.row_seg = np.full((heads, 0, cap), -1, np.int32)
        self.seg_top = 0
        self.free = []            # LIFO list of released segment ids
        self.data = {name: {} for name in fields}  # field -> {segment id -> value}
        self.fields = fields

    def resize(self, V):
        if V <= self.V:
            return
        H, cap = self.H, self.cap
        st = np.zeros((H, V), np.int8)
        off = np.zeros((H, V), np.int32)
        seg = np.full((H, V, cap), -1, np.int32)
        st[:, : self.V] = self.row_state
        off[:, : self.V] = self.row_offset
        seg[:, : self.V] = self.row_seg
        self.row_state, self.row_offset, self.row_seg, self.V = st, off, seg, V

    def alloc(self, n):
        """n ids: first the last min(n, |free|) entries of the free list in list order,
        then fresh ids seg_top, seg_top+1, ..."""
        k = min(n, len(self.free))
        take = []
        if k > 0:
            take = self.free[-k:]
            del self.free[-k:]
        fresh = list(range(self.seg_top, self.seg_top + n - k))
        self.seg_top += n - k
        return take + fresh

    def release(self, ids):
        for s in ids:
            for f in self.fields:
                self.data[f].pop(s, None)
        self.free.extend(int(s) for s in ids)

    def used(self):
        return int(self.row_offset.sum())


class VoxelMerger:
    """Voxel KV memory with P pivots and a B-token buffer per (head, voxel)."""

    def __init__(self, heads, dim, init_voxels=1, pivot_cap=4, budget_cap=8,
                 sim_thresh=0.8, replace_thresh=0.8, score_thresh=0.2, dtype="f32",
                 max_buf_slots=None, max_piv_slots=None):
        self.H, self.D, self.P, self.B = heads, dim, pivot_cap, budget_cap
        self.sim_thresh = float(sim_thresh)
        self.replace_thresh = float(replace_thresh)
        self.score_thresh = float(score_thresh)
        self.dtype = dtype
        self.rnd = make_rounder(dtype)
        # Optional pool bounds (not in the reference's Python path, which grows without limit):
        # rows that would open buffer columns / need a pivot segment beyond the bound are skipped
        # in (head, voxel) order and their selected tokens dropped.
        self.max_buf_slots, self.max_piv_slots = max_buf_slots, max_piv_slots
        self.dropped = 0
        self.V_alloc = max(1, int(init_voxels))
        self.V_used = 0
        self.token_count = 0
        self.buf = SegmentPool(heads, budget_cap, ("K", "V", "S"))
        self.piv = SegmentPool(heads, pivot_cap, ("K", "V", "W", "S", "C"))
        self.buf.resize(self.V_alloc)
        self.piv.resize(self.V_alloc)
        # overflow carried to the next call, in emission order
        self.over = []  # list of (h, v, K, V, S)

    # ------------------------------------------------------------------ capacity
    def ensure_capacity(self, V_needed):
        self.V_used = max(self.V_used, int(V_needed))
        if V_needed <= self.V_alloc:
            return
        V_new = max(int(V_needed), int(self.V_alloc * 1.5))
        while V_new < V_needed:
            V_new = int(V_new * 1.5)
        self.V_alloc = V_new
        self.buf.resize(V_new)
        self.piv.resize(V_new)

    # ------------------------------------------------------------------ helpers
    def _normalize32(self, x):
        n = np.float32(np.sqrt(np.sum(x * x, dtype=np.float32)))
        return x / max(n, np.float32(1e-6))

    def _row_pivots(self, h, v):
        """Valid pivots of a row as lists indexed by slot."""
        n = int(self.piv.row_offset[h, v])
        segs = [int(s) for s in self.piv.row_seg[h, v, :n]]
        return n, segs

    # ------------------------------------------------------------------ insert
    def insert_and_merge(self, K_new, V_new, S_new, VX_new, num_voxels):
        """K_new/V_new [H,T,D], S_new [H,T] float32, VX_new [H,T] int voxel ids."""
        H, T, D = K_new.shape
        assert H == self.H and D == self.D
        if T == 0:
            return
        self.token_count += H * T
        self.ensure_capacity(num_voxels)
        VX_new = np.asarray(VX_new)
        valid = (VX_new >= 0) & (VX_new < self.V_used)
        if not valid.any():
            return
        K_new, V_new, S_new = f32(K_new), f32(V_new), f32(S_new)

        # per-row token lists in processing order: new tokens (ascending position within
        # a head) first, carried overflow after them
        rows = {}
        for h in range(H):
            idx = np.nonzero(valid[h])[0]
            order = idx[np.argsort(VX_new[h, idx], kind="stable")]
            for t in order:
                rows.setdefault((h, int(VX_new[h, t])), []).append(
                    (K_new[h, t], V_new[h, t], np.float32(S_new[h, t])))
        for (h, v, k, val, s) in self.over:
            rows.setdefault((h, v), []).append((k, val, s))
        keys_sorted = sorted(rows.keys())

        # ---- 1. tokens of rows that already hold pivots: merge or select
        selected = {}   # row -> tokens that go on to the buffer
        for key in keys_sorted:
            h, v = key
            toks = rows[key]
            if self.piv.row_state[h, v] == RESERVED:
                selected[key] = toks
                continue
            low = self._merge_into_pivots(h, v, toks)
            keep = [t for t, m in zip(toks, low) if m]
            if keep:
                selected[key] = keep

        # ---- 2. Top-B append; overflow replaces the carried list
        sel_rows = sorted(selected.keys())
        new_over = []
        plans = []
        total_add = 0
        for key in sel_rows:
            h, v = key
            st = self.buf.row_state[h, v]
            if st not in (RESERVED, AVAILABLE):
                raise AssertionError("buffer row is FULL at entry; not reachable in this flow")
            n_old = int(self.buf.row_offset[h, v])
            old = [(self.buf.data["K"][int(s)], self.buf.data["V"][int(s)], self.buf.data["S"][int(s)])
                   for s in self.buf.row_seg[h, v, :n_old]]
            cand = old + [(self.rnd(k), self.rnd(val), s) for (k, val, s) in selected[key]]
            scores = np.array([c[2] for c in cand], np.float32)
            order = np.argsort(-scores, kind="stable")  # score descending, earlier candidate first
            kept = [cand[i] for i in order[: self.B]]
            spill = [cand[i] for i in order[self.B:]]
            add = len(kept) - n_old
            plans.append((key, kept, spill, n_old, add))
            total_add += add
        if self.max_buf_slots is not None or self.max_piv_slots is not None:
            avail_buf = (len(self.buf.free) + self.max_buf_slots - self.buf.seg_top
                         if self.max_buf_slots is not None else None)
            avail_piv = self.max_piv_slots - self.piv.seg_top if self.max_piv_slots is not None else None
            short = ((avail_buf is not None and total_add > avail_buf) or
                     (avail_piv is not None and sum(1 for (key, kept, _, _, _) in plans
                                                    if len(kept) == self.B and self.piv.row_offset[key] < self.P)
                      > avail_piv))
            if short:
                cum_add = cum_piv = 0
                trimmed = []
                for (key, kept, spill, n_old, add) in plans:
                    needs_piv = len(kept) == self.B and self.piv.row_offset[key] < self.P
                    no_buf = avail_buf is not None and add > 0 and cum_add + add > avail_buf
                    no_piv = avail_piv is not None and needs_piv and cum_piv + 1 > avail_piv
                    cum_add += add
                    cum_piv += 1 if needs_piv else 0
                    if no_buf or no_piv:
                        self.dropped += len(selected[key])
                        continue
                    trimmed.append((key, kept, spill, n_old, add))
                plans = trimmed
                total_add = sum(pl[4] for pl in plans)
                sel_rows = [pl[0] for pl in plans]
        ids = self.buf.alloc(total_add)
        cursor = 0
        for key, kept, spill, n_old, add in plans:
            h, v = key
            for c in range(n_old, n_old + add):
                self.buf.row_seg[h, v, c] = ids[cursor]
                cursor += 1
            for c, (k, val, s) in enumerate(kept):
                sid = int(self.buf.row_seg[h, v, c])
                self.buf.data["K"][sid] = k
                self.buf.data["V"][sid] = val
                self.buf.data["S"][sid] = np.float32(s)
            self.buf.row_offset[h, v] = len(kept)
            self.buf.row_state[h, v] = FULL if len(kept) == self.B else AVAILABLE
            for (k, val, s) in spill:
                new_over.append((h, v, k, val, np.float32(s)))
        self.over = new_over

        # ---- 3. full buffers -> one new pivot each, then release the buffer rows
        full = [key for key in sel_rows if self.buf.row_state[key] == FULL]
        packs = [self._cluster_to_pivot(h, v) for (h, v) in full]
        need = sum(1 for (h, v) in full if self.piv.row_offset[h, v] < self.P)
        piv_ids = self.piv.alloc(need)
        cursor = 0
        for (h, v), pack in zip(full, packs):
            n = int(self.piv.row_offset[h, v])
            if n < self.P:
                self.piv.row_seg[h, v, n] = piv_ids[cursor]
                cursor += 1
                slot = n
                self.piv.row_offset[h, v] = n + 1
            else:
                slot = self._evict_victim(h, v)
            sid = int(self.piv.row_seg[h, v, slot])
            for f in ("K", "V", "W", "S", "C"):
                self.piv.data[f][sid] = pack[f]
            cnt = int(self.piv.row_offset[h, v])
            self.piv.row_state[h, v] = FULL if cnt == self.P else AVAILABLE
        freed = []
        for (h, v) in full:
            freed.extend(int(s) for s in self.buf.row_seg[h, v] if s >= 0)
            self.buf.row_seg[h, v] = -1
            self.buf.row_offset[h, v] = 0
            self.buf.row_state[h, v] = RESERVED
        self.buf.release(freed)

    def _merge_into_pivots(self, h, v, toks):
        """Returns per-token flag: True = goes on to the buffer (low similarity, score above gate)."""
        n, segs = self._row_pivots(h, v)
        pd = self.piv.data
        Kp = [f32(pd["K"][s]).copy() for s in segs]
        Vp = [f32(pd["V"][s]).copy() for s in segs]
        Wp = [np.float32(pd["W"][s]) for s in segs]
        Sp = [np.float32(pd["S"][s]) for s in segs]
        Cp = [np.float32(pd["C"][s]) for s in segs]
        Kn = [self._normalize32(k) for k in Kp]
        D = self.D
        accK = [np.zeros(D, np.float32) for _ in range(n)]
        accV = [np.zeros(D, np.float32) for _ in range(n)]
        accA = [np.float32(0)] * n
        accS = [np.float32(0)] * n
        accC = [np.float32(0)] * n
        sim_max = []
        s_clamped = []
        for (k, val, s) in toks:
            s = max(np.float32(s), np.float32(1e-6))
            kn = self._normalize32(f32(k))
            sims = [np.float32(min(1.0, max(-1.0, np.float32(np.dot(kn, Kn[p]))))) for p in range(n)]
            best = int(np.argmax(sims))  # first index on ties
            sm = sims[best]
            sim_max.append(sm)
            s_clamped.append(s)
            if sm >= np.float32(self.sim_thresh):
                a = np.float32(np.exp(sm))
                accK[best] = accK[best] + a * f32(k)
                accV[best] = accV[best] + a * f32(val)
                accA[best] = np.float32(accA[best] + a)
                accS[best] = np.float32(accS[best] + s)
                accC[best] = np.float32(accC[best] + np.float32(1))
        for p in range(n):
            if accA[p] > 0:
                denom = max(np.float32(Wp[p] + accA[p]), np.float32(1e-8))
                Kp[p] = (Wp[p] / denom) * Kp[p] + (np.float32(1.0) / denom) * accK[p]
                Vp[p] = (Wp[p] / denom) * Vp[p] + (np.float32(1.0) / denom) * accV[p]
                Wp[p] = denom
                Sp[p] = np.float32(Sp[p] + accS[p])
                Cp[p] = np.float32(Cp[p] + accC[p])
                sid = segs[p]
                pd["K"][sid] = self.rnd(Kp[p])
                pd["V"][sid] = self.rnd(Vp[p])
                pd["W"][sid], pd["S"][sid], pd["C"][sid] = Wp[p], Sp[p], Cp[p]
        sumS = np.float32(0)
        sumC = np.float32(0)
        for p in range(n):
            sumS = np.float32(sumS + Sp[p])
            sumC = np.float32(sumC + Cp[p])
        gate = np.float32(sumS / max(sumC, np.float32(1e-6))) * np.float32(self.score_thresh)
        return [(sm < np.float32(self.replace_thresh)) and (s > gate)
                for sm, s in zip(sim_max, s_clamped)]

    def _cluster_to_pivot(self, h, v):
        """B buffered tokens -> one pivot, weights exp(cos(k, seed)), seed = first max score."""
        segs = [int(s) for s in self.buf.row_seg[h, v, : self.B]]
        K = np.stack([f32(self.buf.data["K"][s]) for s in segs])
        Vv = np.stack([f32(self.buf.data["V"][s]) for s in segs])
        S = np.maximum(np.array([self.buf.data["S"][s] for s in segs], np.float32), np.float32(1e-6))
        Kn = np.stack([self._normalize32(k) for k in K])
        seed = int(np.argmax(S))
        sim = np.clip((Kn * Kn[seed][None, :]).sum(axis=1, dtype=np.float32), -1.0, 1.0).astype(np.float32)
        w = np.exp(sim).astype(np.float32)
        W = np.float32(w.sum(dtype=np.float32))
        cn = w / (W + np.float32(1e-8))
        return {
            "K": self.rnd((cn[:, None] * K).sum(axis=0, dtype=np.float32)),
            "V": self.rnd((cn[:, None] * Vv).sum(axis=0, dtype=np.float32)),
            "W": W,
            "S": np.float32(S.sum(dtype=np.float32)),
            "C": np.float32(self.B),
        }

    def _evict_victim(self, h, v):
        """Row holds P pivots: fold the lowest-W pivot into its most similar neighbour and
        return the freed slot.  The cosine matrix is computed in the pool dtype, as the
        reference does (stac/merger.py:493-517)."""
        P = self.P
        segs = [int(s) for s in self.piv.row_seg[h, v, :P]]
        pd = self.piv.data
        W = np.array([pd["W"][s] for s in segs], np.float32)
        j = int(np.argmin(W))
        K = np.stack([f32(pd["K"][s]) for s in segs])
        if self.dtype == "bf16":
            nrm = bf16_round(np.sqrt((K * K).sum(axis=1, dtype=np.float32)))
            nrm = np.maximum(nrm, bf16_round(np.float32(1e-6)))
            Kn = bf16_round(K / nrm[:, None])
            sim = bf16_round((Kn * Kn[j][None, :]).sum(axis=1, dtype=np.float32))
        else:
            Kn = np.stack([self._normalize32(k) for k in K])
            sim = (Kn * Kn[j][None, :]).sum(axis=1, dtype=np.float32)
        sim = sim.copy()
        sim[j] = -np.inf
        nb = int(np.argmax(sim))
        if self.dtype == "bf16":
            scale = f32(bf16_round(np.exp(bf16_round(sim[nb] - np.float32(1.0)))))
        else:
            scale = np.float32(np.exp(np.float32(sim[nb] - np.float32(1.0))))
        Wj = np.float32(W[j] * scale)
        Wk = W[nb]
        denom = max(np.float32(Wj + Wk), np.float32(1e-8))
        fj, fk = np.float32(Wj / denom), np.float32(Wk / denom)
        sj, sk = segs[j], segs[nb]
        pd["K"][sk] = self.rnd(fj * f32(pd["K"][sj]) + fk * f32(pd["K"][sk]))
        pd["V"][sk] = self.rnd(fj * f32(pd["V"][sj]) + fk * f32(pd["V"][sk]))
        pd["W"][sk] = denom
        pd["S"][sk] = np.float32(pd["S"][sj] + pd["S"][sk])
        pd["C"][sk] = np.float32(pd["C"][sj] + pd["C"][sk])
        return j

    # ------------------------------------------------------------------ retrieve
    def retrieve(self, voxel_ids=None, retrieve_size=None, return_buf=False):
        """Returns K [H,R,D], V [H,R,D], mask [H,R] bool, bias [H,R] float32 and, for the
        tests, idx [H,R,2] int32 = (voxel, pivot slot) of each valid entry (-1 when padded)."""
        H, P, D = self.H, self.P, self.D
        if voxel_ids is None:
            voxel_ids = np.arange(self.V_used, dtype=np.int64)
        vid = np.unique(np.asarray(voxel_ids, np.int64))
        vid = vid[(vid >= 0) & (vid < self.V_used)]
        req = int(retrieve_size) if retrieve_size is not None else -1
        R = vid.size * P if req <= 0 else req
        K = np.zeros((H, R, D), np.float32)
        Vv = np.zeros((H, R, D), np.float32)
        M = np.zeros((H, R), bool)
        Bz = np.full((H, R), -np.inf, np.float32)
        idx = np.full((H, R, 2), -1, np.int32)
        any_piv = False
        for h in range(H):
            cand = []
            for v in vid:
                n = int(self.piv.row_offset[h, v])
                for p in range(n):
                    sid = int(self.piv.row_seg[h, v, p])
                    cand.append((np.float32(self.piv.data["W"][sid]), int(v), p, sid))
            if not cand:
                continue
            any_piv = True
            w = np.array([c[0] for c in cand], np.float32)
            order = np.argsort(-w, kind="stable")
            for r, i in enumerate(order[:R]):
                _, v, p, sid = cand[i]
                K[h, r] = self.piv.data["K"][sid]
                Vv[h, r] = self.piv.data["V"][sid]
                M[h, r] = True
                Bz[h, r] = np.log(max(np.float32(self.piv.data["C"][sid]), np.float32(1e-9)))
                idx[h, r] = (v, p)
        if not any_piv or not return_buf or req > 0:
            return K, Vv, M, Bz, idx
        # unbounded mode with buffers: append live buffer tokens, (voxel asc, column asc), bias 0
        lists = []
        for h in range(H):
            toks = []
            for v in vid:
                n = int(self.buf.row_offset[h, v])
                for c in range(n):
                    toks.append(int(self.buf.row_seg[h, v, c]))
            lists.append(toks)
        Rb = max(len(t) for t in lists)
        if Rb <= 0:
            return K, Vv, M, Bz, idx
        Kb = np.zeros((H, Rb, D), np.float32)
        Vb = np.zeros((H, Rb, D), np.float32)
        Mb = np.zeros((H, Rb), bool)
        Bb = np.full((H, Rb), -np.inf, np.float32)
        ib = np.full((H, Rb, 2), -1, np.int32)
        for h, toks in enumerate(lists):
            for r, sid in enumerate(toks):
                Kb[h, r] = self.buf.data["K"][sid]
                Vb[h, r] = self.buf.data["V"][sid]
                Mb[h, r] = True
                Bb[h, r] = 0.0
        return (np.concatenate([K, Kb], 1), np.concatenate([Vv, Vb], 1),
                np.concatenate([M, Mb], 1), np.concatenate([Bz, Bb], 1),
                np.concatenate([idx, ib], 1))

    # ------------------------------------------------------------------ snapshots
    def slot_map(self):
        """The graded slot map: state, occupancy and segment ids of both pools over the
        used voxels."""
        V = self.V_used
        return {
            "buf_state": self.buf.row_state[:, :V].copy(),
            "buf_offset": self.buf.row_offset[:, :V].copy(),
            "buf_seg": self.buf.row_seg[:, :V].copy(),
            "piv_state": self.piv.row_state[:, :V].copy(),
            "piv_offset": self.piv.row_offset[:, :V].copy(),
            "piv_seg": self.piv.row_seg[:, :V].copy(),
            "buf_top": self.buf.seg_top, "piv_top": self.piv.seg_top,
            "buf_free": np.array(self.buf.free, np.int32),
        }

    def dense(self):
        """Dense copies of pool contents indexed [H, V_used, slot, ...] for value checks."""
        H, V, P, B, D = self.H, self.V_used, self.P, self.B, self.D
        out = {
            "piv_K": np.zeros((H, V, P, D), np.float32), "piv_V": np.zeros((H, V, P, D), np.float32),
            "piv_W": np.zeros((H, V, P), np.float32), "piv_S": np.zeros((H, V, P), np.float32),
            "piv_C": np.zeros((H, V, P), np.float32),
            "buf_K": np.zeros((H, V, B, D), np.float32), "buf_V": np.zeros((H, V, B, D), np.float32),
            "buf_S": np.zeros((H, V, B), np.float32),
        }
        for h in range(H):
            for v in range(V):
                for p in range(int(self.piv.row_offset[h, v])):
                    sid = int(self.piv.row_seg[h, v, p])
                    for f in ("K", "V", "W", "S", "C"):
                        out["piv_" + f][h, v, p] = self.piv.data[f][sid]
                for c in range(int(self.buf.row_offset[h, v])):
                    sid = int(self.buf.row_seg[h, v, c])
                    for f in ("K", "V", "S"):
                        out["buf_" + f][h, v, c] = self.buf.data[f][sid]
        return out

    def overflow_arrays(self):
        n = len(self.over)
        hv = np.array([(h, v) for (h, v, _, _, _) in self.over], np.int64).reshape(n, 2)
        K = np.stack([o[2] for o in self.over]) if n else np.zeros((0, self.D), np.float32)
        Vv = np.stack([o[3] for o in self.over]) if n else np.zeros((0, self.D), np.float32)
        S = np.array([o[4] for o in self.over], np.float32)
        return hv, K, Vv, S
