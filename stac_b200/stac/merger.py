"""Voxel KV memory behind the reference's ``VoxelKVMerger`` interface (stac/merger.py:50-1602)
with the production allocator (``allocator="segment"``, ``seg_size=1``).

The object owns the pool tensors (the reference's MergerWrapper pattern,
merger-cuda/csrc/merger_wrapper.h:4-9): segment storage for buffered tokens and pivots, the
row -> segment maps, the free list and the carried overflow lists.  All arithmetic happens in
libstac_b200.so (stac_merge_insert, stac_retrieve); this class sizes the arrays, keeps their
pointers in a ``stac_pool`` struct and reads the pool counters back after each insert.
"""

import ctypes

import torch

from .. import _lib
from .._lib import META_BUF_FREE_LEN, META_BUF_TOP, META_BUF_USED, META_OVER_COUNT, META_PIV_TOP, META_PIV_USED
from .._lib import StacEvicted, StacPool, check, ptr, stream_ptr
from ..ops import DeviceStatus, LaggedInts

MAX_LIST = 1 << 22        # STAC_MERGE_MAX_LIST


class VoxelKVMerger:
    def __init__(self, num_heads: int, head_dim: int, init_voxels: int = 0, pivot_cap: int = 4,
                 budget_cap: int = 32, sim_thresh: float = 0.75, replace_thresh: float = 0.5,
                 score_thresh: float = 0.2, dtype: torch.dtype = torch.float16,
                 device=torch.device("cuda"), weight_fn=None, backend: str = "cuda", status=None, **kwargs):
        if head_dim != 64:
            raise ValueError("the sm_100a voxel memory supports head_dim 64 only")
        if not (1 <= int(pivot_cap) <= 4 and 1 <= int(budget_cap) <= 8):
            raise ValueError("supported capacities: pivot_cap <= 4, budget_cap <= 8 "
                             f"(got {pivot_cap}, {budget_cap})")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("pool dtype must be bfloat16 or float32")
        if weight_fn is not None:
            raise ValueError("custom weight_fn is not supported; the merge weight is exp(similarity)")
        alloc = kwargs.get("allocator", "segment")
        if alloc != "segment" or int(kwargs.get("seg_size", 1)) != 1:
            # the other allocators of the reference differ only in slot numbering
            self._alloc_note = f"allocator={alloc!r} mapped to segment/seg_size=1"
        assert replace_thresh <= sim_thresh
        self.H, self.D, self.P, self.B = int(num_heads), int(head_dim), int(pivot_cap), int(budget_cap)
        self.dtype, self.device = dtype, torch.device(device)
        self.debug = kwargs.get("debug", False)
        self.backend = backend
        self.sim_threshold = float(sim_thresh)
        self.replace_threshold = float(replace_thresh)
        self.score_threshold = float(score_thresh)
        self._voxel_alloc = max(1, int(init_voxels))
        self._voxel_offset = 0
        self._token_count = 0
        self._status = status
        self._slab_cap = int(kwargs.get("slab_cap", 1024))
        # optional bounds on the two segment pools (tokens / pivots); None = grow as needed like
        # the reference's Python path.  When a bound is hit, rows are skipped in (head, voxel)
        # order and their tokens dropped (counted in info()["dropped_tokens"]).
        self._max_buf = kwargs.get("max_buffer_slots", None)
        self._max_piv = kwargs.get("max_pivot_slots", None)
        if (self._max_buf is not None and self._max_buf < 1) or (self._max_piv is not None and self._max_piv < 1):
            raise ValueError("pool bounds must be positive")
        dev = self.device
        H, P, B, D = self.H, self.P, self.B, self.D
        V = self._voxel_alloc
        self._buf_row_seg = torch.full((H, V, B), -1, dtype=torch.int32, device=dev)
        self._buf_row_cnt = torch.zeros((H, V), dtype=torch.int32, device=dev)
        self._piv_row_seg = torch.full((H, V, P), -1, dtype=torch.int32, device=dev)
        self._piv_row_cnt = torch.zeros((H, V), dtype=torch.int32, device=dev)
        self._buf_cap = 0
        self._piv_cap = 0
        self._buf_K = self._buf_V = self._buf_S = self._buf_free = None
        self._piv_K = self._piv_V = self._piv_W = self._piv_S = self._piv_C = None
        self._grow_buf(min(max(1024, self._slab_cap * B), int(self._max_buf) if self._max_buf else 1 << 62))
        self._grow_piv(min(max(1024, V), int(self._max_piv) if self._max_piv else 1 << 62))
        self._over = [self._new_over(1), self._new_over(1)]
        self._over_cur = 0
        self._over_cap = 1
        self._meta = torch.zeros(_lib.META_SIZE, dtype=torch.int32, device=dev)
        self._meta_host = [0] * _lib.META_SIZE
        self._over_max_head = 0
        self._voxel_count_dev = None     # device scalar with the table's voxel count (set by the manager)
        # counters, overflow offsets and the status word of the last insert, read one call late
        self._mirror = LaggedInts(_lib.META_SIZE + self.H + 1 + 1)
        self._scratch = None
        self._ret_sel = None

    # ------------------------------------------------------------------ storage
    def _new_over(self, cap):
        dev = self.device
        return {"K": torch.empty((cap, self.D), dtype=self.dtype, device=dev),
                "V": torch.empty((cap, self.D), dtype=self.dtype, device=dev),
                "S": torch.empty(cap, dtype=torch.float32, device=dev),
                "hv": torch.empty((cap, 2), dtype=torch.int32, device=dev),
                "start": torch.zeros(self.H + 1, dtype=torch.int32, device=dev)}

    @staticmethod
    def _extend(old, shape, dtype, device, fill=None):
        new = torch.empty(shape, dtype=dtype, device=device) if fill is None else \
            torch.full(shape, fill, dtype=dtype, device=device)
        if old is not None and old.numel() > 0:
            new[: old.shape[0]].copy_(old)
        return new

    def _grow_buf(self, cap):
        if cap <= self._buf_cap:
            return
        dev = self.device
        self._buf_K = self._extend(self._buf_K, (cap, self.D), self.dtype, dev)
        self._buf_V = self._extend(self._buf_V, (cap, self.D), self.dtype, dev)
        self._buf_S = self._extend(self._buf_S, (cap,), torch.float32, dev)
        self._buf_free = self._extend(self._buf_free, (cap,), torch.int32, dev)
        self._buf_cap = cap

    def _grow_piv(self, cap):
        if cap <= self._piv_cap:
            return
        dev = self.device
        self._piv_K = self._extend(self._piv_K, (cap, self.D), self.dtype, dev)
        self._piv_V = self._extend(self._piv_V, (cap, self.D), self.dtype, dev)
        self._piv_W = self._extend(self._piv_W, (cap,), torch.float32, dev)
        self._piv_S = self._extend(self._piv_S, (cap,), torch.float32, dev)
        self._piv_C = self._extend(self._piv_C, (cap,), torch.float32, dev)
        self._piv_cap = cap

    def _grow_rows(self, V_new):
        dev = self.device
        H, P, B = self.H, self.P, self.B
        V_old = self._buf_row_cnt.shape[1]
        if V_new <= V_old:
            return
        # rows cost 56 bytes per (head, voxel): grow by the reference's x1.5 rule, not faster
        brs = torch.full((H, V_new, B), -1, dtype=torch.int32, device=dev)
        brc = torch.zeros((H, V_new), dtype=torch.int32, device=dev)
        prs = torch.full((H, V_new, P), -1, dtype=torch.int32, device=dev)
        prc = torch.zeros((H, V_new), dtype=torch.int32, device=dev)
        brs[:, :V_old].copy_(self._buf_row_seg)
        brc[:, :V_old].copy_(self._buf_row_cnt)
        prs[:, :V_old].copy_(self._piv_row_seg)
        prc[:, :V_old].copy_(self._piv_row_cnt)
        self._buf_row_seg, self._buf_row_cnt, self._piv_row_seg, self._piv_row_cnt = brs, brc, prs, prc

    def reset(self):
        pass

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        """Everything a later insert / retrieve depends on, cut to the used extents: row maps of
        the used voxels, both pools up to their bump pointers, the free list, the carried-over
        overflow list and the device counters."""
        self._pull_meta()
        m = self._meta_host
        V = self.used_voxels()
        top_b, n_free, top_p, n_over = m[META_BUF_TOP], m[META_BUF_FREE_LEN], m[_lib.META_PIV_TOP], m[META_OVER_COUNT]
        cur = self._over[self._over_cur]
        cpu = lambda t: t.cpu().clone()
        return {
            "voxel_alloc": int(self._voxel_alloc), "voxel_offset": V, "token_count": int(self._token_count),
            "meta": cpu(self._meta), "over_max_head": int(self._over_max_head),
            "buf_row_seg": cpu(self._buf_row_seg[:, :V]), "buf_row_cnt": cpu(self._buf_row_cnt[:, :V]),
            "piv_row_seg": cpu(self._piv_row_seg[:, :V]), "piv_row_cnt": cpu(self._piv_row_cnt[:, :V]),
            "buf_K": cpu(self._buf_K[:top_b]), "buf_V": cpu(self._buf_V[:top_b]), "buf_S": cpu(self._buf_S[:top_b]),
            "buf_free": cpu(self._buf_free[:n_free]),
            "piv_K": cpu(self._piv_K[:top_p]), "piv_V": cpu(self._piv_V[:top_p]), "piv_W": cpu(self._piv_W[:top_p]),
            "piv_S": cpu(self._piv_S[:top_p]), "piv_C": cpu(self._piv_C[:top_p]),
            "over": {f: cpu(cur[f][:n_over]) for f in ("K", "V", "S", "hv")} | {"start": cpu(cur["start"])},
        }

    def load_state_dict(self, sd):
        """Into a freshly constructed merger of the same configuration."""
        V = int(sd["voxel_offset"])
        self._voxel_alloc = max(int(sd["voxel_alloc"]), self._voxel_alloc)
        self._grow_rows(self._voxel_alloc)
        self._voxel_offset = V
        self._token_count = int(sd["token_count"])
        for name in ("buf_row_seg", "buf_row_cnt", "piv_row_seg", "piv_row_cnt"):
            getattr(self, "_" + name)[:, :V].copy_(sd[name])
        top_b, n_free, top_p = sd["buf_K"].shape[0], sd["buf_free"].shape[0], sd["piv_K"].shape[0]
        self._grow_buf(max(top_b, n_free, 1))
        self._grow_piv(max(top_p, 1))
        for name in ("buf_K", "buf_V", "buf_S"):
            getattr(self, "_" + name)[:top_b].copy_(sd[name])
        self._buf_free[:n_free].copy_(sd["buf_free"])
        for name in ("piv_K", "piv_V", "piv_W", "piv_S", "piv_C"):
            getattr(self, "_" + name)[:top_p].copy_(sd[name])
        n_over = sd["over"]["S"].shape[0]
        self._over_cap = max(n_over, 1)
        self._over = [self._new_over(self._over_cap), self._new_over(self._over_cap)]
        self._over_cur = 0
        for f in ("K", "V", "S", "hv"):
            self._over[0][f][:n_over].copy_(sd["over"][f])
        self._over[0]["start"].copy_(sd["over"]["start"])
        self._meta.copy_(sd["meta"])
        self._meta_host = sd["meta"].tolist()
        self._over_max_head = int(sd["over_max_head"])

    def update_voxel_zones(self, voxel_zones):
        """Morton zones only steer the reference's CUDA pivot allocator; nothing to do here."""

    def ensure_capacity(self, V_needed: int):
        """Voxel rows grow by x1.5 as in stac/merger.py:218-239."""
        self._voxel_offset = max(int(V_needed), self._voxel_offset)
        if V_needed <= self._voxel_alloc:
            return
        V_new = max(int(V_needed), int(self._voxel_alloc * 1.5))
        while V_new < V_needed:
            V_new = int(V_new * 1.5)
        self._voxel_alloc = V_new
        self._grow_rows(V_new)

    def _pool_struct(self):
        cur, nxt = self._over[self._over_cur], self._over[1 - self._over_cur]
        s = StacPool()
        s.heads, s.head_dim, s.elem_bytes = self.H, self.D, 2 if self.dtype == torch.bfloat16 else 4
        s.pivot_cap, s.budget_cap = self.P, self.B
        s.voxel_cap, s.voxel_used = int(self._buf_row_cnt.shape[1]), int(self._voxel_offset)
        s.sim_thresh, s.replace_thresh, s.score_thresh = (self.sim_threshold, self.replace_threshold,
                                                          self.score_threshold)
        s.buf_K, s.buf_V, s.buf_S = self._buf_K.data_ptr(), self._buf_V.data_ptr(), self._buf_S.data_ptr()
        s.buf_row_seg, s.buf_row_cnt = self._buf_row_seg.data_ptr(), self._buf_row_cnt.data_ptr()
        s.buf_free, s.buf_cap = self._buf_free.data_ptr(), self._buf_cap
        s.piv_K, s.piv_V = self._piv_K.data_ptr(), self._piv_V.data_ptr()
        s.piv_W, s.piv_S, s.piv_C = self._piv_W.data_ptr(), self._piv_S.data_ptr(), self._piv_C.data_ptr()
        s.piv_row_seg, s.piv_row_cnt, s.piv_cap = (self._piv_row_seg.data_ptr(), self._piv_row_cnt.data_ptr(),
                                                   self._piv_cap)
        s.over_K_in, s.over_V_in, s.over_S_in = cur["K"].data_ptr(), cur["V"].data_ptr(), cur["S"].data_ptr()
        s.over_hv_in, s.over_start_in = cur["hv"].data_ptr(), cur["start"].data_ptr()
        s.over_K_out, s.over_V_out, s.over_S_out = nxt["K"].data_ptr(), nxt["V"].data_ptr(), nxt["S"].data_ptr()
        s.over_hv_out, s.over_start_out = nxt["hv"].data_ptr(), nxt["start"].data_ptr()
        s.over_cap = self._over_cap
        s.meta = self._meta.data_ptr()
        s.voxel_count = self._voxel_count_dev.data_ptr() if self._voxel_count_dev is not None else None
        return s

    def _push_meta(self):
        """Enqueue the copy of the pool counters, the per-head overflow offsets and the status word
        to pinned host memory behind the insert that produced them; nothing waits here."""
        word = self._status.word if self._status is not None else torch.zeros(1, dtype=torch.int32, device=self.device)
        self._mirror.push(self._meta, self._over[self._over_cur]["start"], word)

    def _pull_meta(self):
        """Take in what the last insert left behind (waits for that insert if it is still running);
        a device-side error of that insert is raised here."""
        vals = self._mirror.pull()
        if vals is None:
            return
        n = _lib.META_SIZE
        self._meta_host = vals[:n]
        start = vals[n:n + self.H + 1]
        self._over_max_head = max((b - a for a, b in zip(start[:-1], start[1:])), default=0)
        code = vals[n + self.H + 1]
        if code != 0 and self._status is not None:
            self._status.clear()
            raise _lib.StacError(f"voxel merge: device error {code} ({DeviceStatus.NAMES.get(code, 'unknown')})")

    # ------------------------------------------------------------------ insert
    @torch.no_grad()
    def insert_evicted(self, k_cache, v_cache, scores, voxel_ids, positions, tokens_per_head, num_voxels,
                       voxel_count_dev=None):
        """Evicted tokens read in place: token j of pool head h sits at position
        positions[h, j] of k_cache/v_cache [H, T, D], scores/voxel_ids [H, T]
        (positions None = the first tokens_per_head positions).  `num_voxels` may be an upper
        bound of the voxel count if `voxel_count_dev` (int32 device scalar with the exact count)
        is given: the bound sizes the row arrays, the exact count is recorded on the device."""
        self._voxel_count_dev = voxel_count_dev
        H, D = self.H, self.D
        Tn = int(tokens_per_head)
        if Tn == 0:
            return
        assert k_cache.dtype == self.dtype and v_cache.dtype == self.dtype
        assert k_cache.stride(-1) == 1 and k_cache.stride(1) == D and v_cache.stride() == k_cache.stride()
        assert scores.dtype == torch.float32 and voxel_ids.dtype == torch.int32
        assert scores.stride(1) == 1 and voxel_ids.stride() == scores.stride()
        self._pull_meta()                 # counters of the previous insert (a whole step old)
        self._token_count += H * Tn
        self.ensure_capacity(num_voxels)
        over_in = self._meta_host[META_OVER_COUNT]
        E = H * Tn + over_in
        # worst-case needs of this call (see the capacity notes in the module docstring)
        need_buf = self._meta_host[META_BUF_TOP] + max(0, E - self._meta_host[META_BUF_FREE_LEN])
        if self._max_buf is not None:
            need_buf = min(need_buf, max(int(self._max_buf), self._buf_cap))
        if need_buf > self._buf_cap:
            grow = max(need_buf, int(self._buf_cap * 1.5))
            self._grow_buf(grow if self._max_buf is None else min(grow, max(int(self._max_buf), need_buf)))
        need_piv = self._meta_host[META_PIV_TOP] + (self._meta_host[META_BUF_USED] + E) // self.B + 1
        if self._max_piv is not None:
            need_piv = min(need_piv, max(int(self._max_piv), self._piv_cap))
        if need_piv > self._piv_cap:
            grow = max(need_piv, int(self._piv_cap * 1.5))
            self._grow_piv(grow if self._max_piv is None else min(grow, max(int(self._max_piv), need_piv)))
        if E > self._over_cap:
            cap = max(E, int(self._over_cap * 1.5))
            cur = self._over[self._over_cur]
            new_cur = self._new_over(cap)
            n = over_in
            for f in ("K", "V", "S", "hv"):
                new_cur[f][:n].copy_(cur[f][:n])
            new_cur["start"].copy_(cur["start"])
            self._over[self._over_cur] = new_cur
            self._over[1 - self._over_cur] = self._new_over(cap)
            self._over_cap = cap
        ncap = Tn + self._over_max_head
        ncap = (ncap + 2047) // 2048 * 2048        # few distinct scratch sizes
        if ncap > MAX_LIST:
            raise _lib.StacError(f"{ncap} tokens for one pool head in one call; the limit is {MAX_LIST}")
        need = _lib.lib().stac_merge_scratch_bytes(H, ncap, self._buf_cap)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(int(need * 1.5), dtype=torch.uint8, device=self.device)
        pool = self._pool_struct()
        ev = StacEvicted()
        ev.k, ev.v = k_cache.data_ptr(), v_cache.data_ptr()
        ev.kv_head_stride, ev.kv_row_stride = k_cache.stride(0), k_cache.stride(1)
        ev.scores, ev.voxel_ids = scores.data_ptr(), voxel_ids.data_ptr()
        ev.meta_head_stride = scores.stride(0)
        ev.positions = positions.data_ptr() if positions is not None else None
        ev.tokens_per_head = Tn
        if positions is not None:
            assert positions.dtype == torch.int32 and positions.is_contiguous()
            assert tuple(positions.shape) == (H, Tn)
        st = _lib.lib().stac_merge_insert(ctypes.byref(pool), ctypes.byref(ev), ptr(self._scratch),
                                          self._scratch.numel(), ncap,
                                          ptr(self._status.word) if self._status is not None else None,
                                          stream_ptr())
        check(st, "stac_merge_insert")
        self._over_cur = 1 - self._over_cur
        self._push_meta()

    @torch.no_grad()
    def insert_and_merge(self, K_new, V_new, S_new, I_new, VX_new, num_voxels: int, mode: str = "default"):
        """Reference signature (stac/merger.py:1157-1255): K_new/V_new [H,Tn,D], S_new [H,Tn]
        fp32, I_new ignored, VX_new [H,Tn] voxel ids."""
        H, Tn, D = K_new.shape
        assert H == self.H and D == self.D
        assert V_new.shape == K_new.shape and S_new.shape == VX_new.shape == (H, Tn)
        if Tn == 0:
            return {}
        self.insert_evicted(K_new.to(self.dtype).contiguous(), V_new.to(self.dtype).contiguous(),
                            S_new.to(torch.float32).contiguous(), VX_new.to(torch.int32).contiguous(),
                            None, Tn, num_voxels)
        return {"init_time": 0.0, "append_time": 0.0, "merge_all2one_time": 0.0, "merge_one2one_time": 0.0}

    # ------------------------------------------------------------------ retrieve
    @torch.no_grad()
    def retrieve_device(self, query_ids, query_count, retrieve_size, want_idx=False):
        """query_ids int32 ascending (device), query_count int32 [1] (device).  Returns
        K, V [H,R,D], mask bool [H,R], bias fp32 [H,R] (and idx int32 [H,R,2])."""
        R = int(retrieve_size)
        if not (0 < R <= 8192):
            raise ValueError("retrieve_size must be in 1..8192")
        dev = self.device
        K = torch.empty((self.H, R, self.D), dtype=self.dtype, device=dev)
        V = torch.empty((self.H, R, self.D), dtype=self.dtype, device=dev)
        M = torch.empty((self.H, R), dtype=torch.uint8, device=dev)
        Bz = torch.empty((self.H, R), dtype=torch.float32, device=dev)
        idx = torch.empty((self.H, R, 2), dtype=torch.int32, device=dev) if want_idx else None
        if self._ret_sel is None or self._ret_sel.numel() < self.H * R:
            self._ret_sel = torch.empty(self.H * R, dtype=torch.int32, device=dev)
        pool = self._pool_struct()
        st = _lib.lib().stac_retrieve(ctypes.byref(pool), ptr(query_ids), ptr(query_count), R,
                                      ptr(self._ret_sel), ptr(K), ptr(V), ptr(M), ptr(Bz), ptr(idx),
                                      stream_ptr())
        check(st, "stac_retrieve")
        out = (K, V, M.bool(), Bz)
        return out + (idx,) if want_idx else out

    @torch.no_grad()
    def retrieve(self, voxel_ids=None, return_buf: bool = False, retrieve_size=None, want_idx=False):
        """Reference signature (stac/merger.py:1377-1543) for retrieve_size > 0: fixed-size
        output, pivots ordered by W descending, bias log C, padding -inf.  With a positive
        retrieve_size the reference never returns buffer tokens, whatever return_buf says."""
        req = int(retrieve_size) if retrieve_size is not None else -1
        dev = self.device
        if req <= 0:
            return self._retrieve_unbounded(voxel_ids, return_buf, want_idx)
        if voxel_ids is None:
            ids = torch.arange(self.used_voxels(), device=dev, dtype=torch.int32)
        else:
            ids = torch.unique(voxel_ids.to(device=dev, dtype=torch.int64))
            ids = ids[(ids >= 0) & (ids < self._voxel_offset)].to(torch.int32).contiguous()
        cnt = torch.tensor([ids.numel()], dtype=torch.int32, device=dev)
        if ids.numel() == 0:
            ids = torch.zeros(1, dtype=torch.int32, device=dev)
        return self.retrieve_device(ids, cnt, req, want_idx)

    @torch.no_grad()
    def _retrieve_unbounded(self, voxel_ids, return_buf, want_idx=False):
        """retrieve_size <= 0 (stac/merger.py:1424-1543): output width = (#queried voxels) * P,
        plus, with return_buf, the buffered tokens of those voxels ((voxel, column) order, bias 0)
        padded to the longest head.  The output size depends on data, so this mode reads counts
        back to the host; it is assembled from the pool tensors with torch indexing ops (device
        plumbing only, no arithmetic beyond log C) and is not on the streaming path, which uses
        a fixed retrieve_size."""
        dev, H, P, B, D = self.device, self.H, self.P, self.B, self.D
        if voxel_ids is None:
            vid = torch.arange(self.used_voxels(), device=dev, dtype=torch.int64)
        else:
            vid = torch.unique(voxel_ids.to(device=dev, dtype=torch.int64))
            vid = vid[(vid >= 0) & (vid < self._voxel_offset)]
        Q = int(vid.numel())
        R = Q * P

        def empty(n):
            return (torch.zeros(H, n, D, dtype=self.dtype, device=dev), torch.zeros(H, n, D, dtype=self.dtype, device=dev),
                    torch.zeros(H, n, dtype=torch.bool, device=dev),
                    torch.full((H, n), float("-inf"), dtype=torch.float32, device=dev),
                    torch.full((H, n, 2), -1, dtype=torch.int32, device=dev))

        def done(t):
            return t if want_idx else t[:4]
        if Q == 0:
            return done(empty(R))
        cnt = self._piv_row_cnt[:, vid]                                   # [H,Q]
        seg = self._piv_row_seg[:, vid, :]                                # [H,Q,P]
        slot = torch.arange(P, device=dev).view(1, 1, P)
        mask = (slot < cnt.unsqueeze(-1)).reshape(H, R)
        if not bool(mask.any()):
            return done(empty(R))
        segf = seg.reshape(H, R).clamp(min=0).long()
        W = torch.where(mask, self._piv_W[segf], torch.zeros((), device=dev))
        order = torch.argsort(W, dim=1, descending=True, stable=True)      # valid pivots first
        segs = torch.gather(segf, 1, order)
        m = torch.gather(mask, 1, order)
        K = self._piv_K[segs] * m.unsqueeze(-1).to(self.dtype)
        V = self._piv_V[segs] * m.unsqueeze(-1).to(self.dtype)
        C = self._piv_C[segs]
        bias = torch.where(m, torch.log(C.clamp_min(1e-9)), torch.full((), float("-inf"), device=dev))
        vox = vid.view(1, Q, 1).expand(H, Q, P).reshape(H, R)
        idx = torch.stack([torch.gather(vox, 1, order), torch.gather(slot.expand(H, Q, P).reshape(H, R), 1, order)], -1)
        idx = torch.where(m.unsqueeze(-1), idx, torch.full((), -1, device=dev, dtype=idx.dtype)).to(torch.int32)
        if not return_buf:
            return done((K, V, m, bias, idx))
        bcnt = self._buf_row_cnt[:, vid]                                   # [H,Q]
        bseg = self._buf_row_seg[:, vid, :].reshape(H, Q * B)
        col = torch.arange(B, device=dev).view(1, 1, B)
        bmask = (col < bcnt.unsqueeze(-1)).reshape(H, Q * B)
        Rb = int(bmask.sum(dim=1).max().item())
        if Rb <= 0:
            return done((K, V, m, bias, idx))
        border = torch.argsort((~bmask).to(torch.int8), dim=1, stable=True)[:, :Rb]   # keeps (voxel, column) order
        bm = torch.gather(bmask, 1, border)
        bs = torch.gather(bseg.clamp(min=0).long(), 1, border)
        Kb = self._buf_K[bs] * bm.unsqueeze(-1).to(self.dtype)
        Vb = self._buf_V[bs] * bm.unsqueeze(-1).to(self.dtype)
        bb = torch.where(bm, torch.zeros((), device=dev), torch.full((), float("-inf"), device=dev))
        ib = torch.full((H, Rb, 2), -1, dtype=torch.int32, device=dev)
        return done((torch.cat([K, Kb], 1), torch.cat([V, Vb], 1), torch.cat([m, bm], 1), torch.cat([bias, bb], 1),
                     torch.cat([idx, ib], 1)))

    # ------------------------------------------------------------------ stats
    def _pool_counts(self):
        self._pull_meta()
        m = self._meta_host
        return m[META_BUF_USED], self._buf_cap, m[META_PIV_USED], self._piv_cap

    def info(self) -> dict:
        buf_data, buf_alloc, piv_data, piv_alloc = self._pool_counts()
        tc = float(self._token_count + 1e-6)
        return dict(head_dim=self.D, num_heads=self.H, pivot_capacity=self.P, buffer_capacity=self.B,
                    used_voxels=self.used_voxels(), allocated_voxels=self._voxel_alloc,
                    token_count=self._token_count, merge_compress_ratio=piv_data / tc,
                    best_compress_ratio=(piv_data + buf_data) / tc,
                    real_compress_ratio=(piv_alloc + buf_alloc) / tc,
                    pivot_pool_used=piv_data, pivot_pool_alloc=piv_alloc,
                    buffer_pool_used=buf_data, buffer_pool_alloc=buf_alloc,
                    dropped_tokens=self._meta_host[_lib.META_DROPPED])

    def used_voxels(self) -> int:
        """Voxels known at the last insert (exact; waits for that insert if need be)."""
        self._pull_meta()
        if self._voxel_count_dev is not None:
            return int(self._meta_host[_lib.META_VOXELS])
        return int(self._voxel_offset)

    def check_status(self):
        """Wait for the last insert and raise if it reported a device-side error."""
        self._pull_meta()

    def memory(self) -> dict:
        buf_data, buf_alloc, piv_data, piv_alloc = self._pool_counts()
        kvb = 2 if self.dtype == torch.bfloat16 else 4
        mb = 1024 ** 2
        return dict(buffer_used_mem=buf_data * (self.D * 2 * kvb + 4) / mb,
                    buffer_alloc_mem=buf_alloc * (self.D * 2 * kvb + 4) / mb,
                    pivot_used_mem=piv_data * (self.D * 2 * kvb + 8) / mb,
                    pivot_alloc_mem=piv_alloc * (self.D * 2 * kvb + 8) / mb)

    # ------------------------------------------------------------------ test hooks
    def snapshot(self):
        """Host copies of the slot maps and pool contents over the used voxels (tests)."""
        self._pull_meta()
        V = self.used_voxels()
        m = self._meta.cpu().tolist()
        cur = self._over[self._over_cur]
        n_over = m[META_OVER_COUNT]
        brs = self._buf_row_seg[:, :V].cpu()
        prs = self._piv_row_seg[:, :V].cpu()

        def gather(pool, seg):
            idx = seg.clamp(min=0).long()
            out = pool.float().cpu()[idx]
            mask = (seg >= 0)
            return out * mask.reshape(mask.shape + (1,) * (out.dim() - mask.dim())).float()

        return {
            "buf_offset": self._buf_row_cnt[:, :V].cpu().numpy(), "buf_seg": brs.numpy(),
            "piv_offset": self._piv_row_cnt[:, :V].cpu().numpy(), "piv_seg": prs.numpy(),
            "buf_top": m[META_BUF_TOP], "piv_top": m[META_PIV_TOP],
            "buf_free": self._buf_free[: m[META_BUF_FREE_LEN]].cpu().numpy(),
            "buf_K": gather(self._buf_K, brs).numpy(), "buf_V": gather(self._buf_V, brs).numpy(),
            "buf_S": gather(self._buf_S, brs).numpy(),
            "piv_K": gather(self._piv_K, prs).numpy(), "piv_V": gather(self._piv_V, prs).numpy(),
            "piv_W": gather(self._piv_W, prs).numpy(), "piv_S": gather(self._piv_S, prs).numpy(),
            "piv_C": gather(self._piv_C, prs).numpy(),
            "over_hv": cur["hv"][:n_over].cpu().numpy().astype("int64"),
            "over_K": cur["K"][:n_over].float().cpu().numpy(), "over_V": cur["V"][:n_over].float().cpu().numpy(),
            "over_S": cur["S"][:n_over].cpu().numpy(),
        }
