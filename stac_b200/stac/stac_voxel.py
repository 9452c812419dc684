"""STAC voxel KV manager behind the reference's ``STACVoxelKV`` interface
(stac/stac_voxel.py:23-980): H2O hot cache + a voxel memory that absorbs evicted tokens and
gives back pivots around the current frames.

Per chunk, in the reference's call order:
  append_kv (per layer) -> decode_sparse_attn (per layer: window + pivot attention, column sums
  -> scores) -> append_positions (points -> voxel ids, neighbour voxels of the recent tokens)
  -> [retrieve_kv] -> prune_kv (H2O keep set, eviction merge into the voxel memory, compaction).
Each step is one or a few kernels of libstac_b200.so.  Nothing on this path waits for the GPU:
the voxel count and the pool counters travel to pinned host memory behind the kernels that
produce them and are taken in by the next call that needs them, one stream step later; until
then the host works with an upper bound of the voxel count (stats getters return exact
numbers and wait if they must).
"""

import logging
from typing import Dict, List, Optional, Tuple

import torch

from .h2o import HeavyHittersKV
from .merger import VoxelKVMerger
from .voxel import BinaryVoxel

logger = logging.getLogger(__name__)


class STACVoxelKV(HeavyHittersKV):
    def __init__(self, *args, voxel_size: float = 0.05, voxelize_layers: Optional[List[int]] = None,
                 init_voxels: int = 1024, voxel_buf_cap: int = 32, voxel_piv_cap: int = 4,
                 voxel_backend: str = "python", sim_threshold: float = 0.8, replace_threshold: float = 0.8,
                 score_threshold: float = 0, weight_fn=None, allocator: str = "slab", slab_growth=256,
                 slab_free_policy="immediate", slab_cap=1024, seg_size: int = 4, alloc_debug: bool = False,
                 retrieval_size: int = -1, enable_alloc_cpu: bool = False, gpu_threshold_gb: float = 10.0,
                 **kwargs):
        super().__init__(*args, **kwargs)
        if voxelize_layers is not None and set(voxelize_layers) != set(range(self.num_layers)):
            raise ValueError("voxelize_layers must be None (all layers) on the sm_100a path")
        if enable_alloc_cpu:
            raise ValueError("enable_alloc_cpu is a dead option in the reference "
                             "(stac/stac_voxel.py:383-385 calls undefined methods) and is not provided")
        self._voxel_size_f = float(voxel_size)
        self._voxel_size = torch.tensor(voxel_size, dtype=torch.float32, device=self.device)
        self._vm = BinaryVoxel(voxel_size=voxel_size, device=self.device)
        self._recent_voxel_ids = None
        self._voxelize_list = [True for _ in range(self.num_layers)]
        # every backend / allocator name of the reference maps to the one native implementation
        self._vk_conf = dict(num_heads=self.num_heads, head_dim=self.head_dim, init_voxels=init_voxels,
                             pivot_cap=voxel_piv_cap, budget_cap=voxel_buf_cap, sim_thresh=sim_threshold,
                             replace_thresh=replace_threshold, score_thresh=score_threshold,
                             weight_fn=weight_fn, dtype=self.dtype, device=self.device, debug=self.debug,
                             allocator=allocator, backend=voxel_backend, slab_growth=slab_growth,
                             slab_free_policy=slab_free_policy, slab_cap=slab_cap, seg_size=seg_size,
                             alloc_debug=alloc_debug,
                             # optional bounds of the voxel memory (extension; None = unbounded)
                             max_buffer_slots=kwargs.get("max_buffer_slots"),
                             max_pivot_slots=kwargs.get("max_pivot_slots"))
        self._enable_alloc_cpu = False
        # the reference overwrites recent_size here after the token sizes were derived
        # (stac/stac_voxel.py:109-110); only log lines read it afterwards
        self.recent_size = retrieval_size
        self.retrieval_token_size = int(retrieval_size * self.token_per_f)
        self._vstore = None

    # ------------------------------------------------------------------ reset / free
    def reset(self):
        super().reset()
        L, H, T = self._L_eff, self.num_heads, self.reserved_buffer_token_size
        dev = self.device
        self._vm._status = self._status
        self._vm.reset()
        self._recent_voxel_ids = None
        conf = dict(self._vk_conf)
        conf["num_heads"] = L * H
        self._vstore = VoxelKVMerger(status=self._status, **conf)
        self._vx = [torch.full((L, H, T), -1, dtype=torch.int32, device=dev) for _ in range(2)]
        self._token_voxel_indices = self._vx[self._cur]
        self._offset_voxel = [0] * L
        self._ret = None
        self.key_cache_retrieval = [torch.empty(H, 0, self.head_dim, device=dev, dtype=self.dtype)
                                    for _ in range(L)]
        self.value_cache_retrieval = [torch.empty(H, 0, self.head_dim, device=dev, dtype=self.dtype)
                                      for _ in range(L)]
        self._bias_retrieval = [torch.empty(H, 0, device=dev, dtype=torch.float32) for _ in range(L)]
        self._scores_retrieval = [torch.zeros(H, 0, device=dev, dtype=torch.float32) for _ in range(L)]
        self._offset_retrieval = [0] * L

    def free(self):
        self._token_voxel_indices = None
        self._vx = None
        self._offset_voxel = [0] * self._L_eff
        self._ret = None
        for l in range(self._L_eff):
            self.key_cache_retrieval[l] = None
            self.value_cache_retrieval[l] = None
            self._bias_retrieval[l] = None
            self._scores_retrieval[l] = None
            self._offset_retrieval[l] = 0
        self._vstore = None
        return super().free()

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        """Hot cache, scores, voxel ids per token, the voxel table, the voxel memory and the
        retrieved pivots that the next attention calls would read."""
        sd = super().state_dict()
        T = max(self._offset_voxel)
        rec = None
        if self._recent_voxel_ids is not None:
            ids, count = self._recent_voxel_ids
            n = int(count.item())
            rec = ids[:n].cpu().clone()
        sd.update(voxel_idx=self._token_voxel_indices[:, :, :T].cpu().clone(), offset_voxel=list(self._offset_voxel),
                  recent_voxel_ids=rec, table=self._vm.state_dict(), memory=self._vstore.state_dict(),
                  retrieved=None if self._ret is None else [t.cpu().clone() for t in self._ret],
                  offset_retrieval=list(self._offset_retrieval),
                  scores_retrieval=[t.cpu().clone() for t in self._scores_retrieval])
        return sd

    def load_state_dict(self, sd):
        super().load_state_dict(sd)          # resets everything, then hot cache and scores
        dev, L, H = self.device, self._L_eff, self.num_heads
        T = sd["voxel_idx"].shape[2]
        self._token_voxel_indices[:, :, :T].copy_(sd["voxel_idx"])
        self._offset_voxel = list(sd["offset_voxel"])
        self._vm.load_state_dict(sd["table"])
        self._vstore.load_state_dict(sd["memory"])
        self._recent_voxel_ids = None
        if sd["recent_voxel_ids"] is not None:
            ids = sd["recent_voxel_ids"].to(dev)
            self._recent_voxel_ids = (ids, torch.tensor([ids.numel()], dtype=torch.int32, device=dev))
        if sd["retrieved"] is not None:
            K, V, M, B = (t.to(dev) for t in sd["retrieved"])
            self._ret = (K, V, M, B)
            for s in range(L):
                Tm = int(sd["offset_retrieval"][s])
                if Tm == 0:
                    continue
                self.key_cache_retrieval[s] = K[s * H:(s + 1) * H, :Tm]
                self.value_cache_retrieval[s] = V[s * H:(s + 1) * H, :Tm]
                self._bias_retrieval[s] = B[s * H:(s + 1) * H, :Tm]
                self._offset_retrieval[s] = Tm
        self._scores_retrieval = [t.to(dev) for t in sd["scores_retrieval"]]

    # ------------------------------------------------------------------ attention
    @torch.no_grad()
    def decode_sparse_attn(self, query_states: torch.Tensor, layer_idx: int) -> torch.Tensor:
        """Attention over [hot | retrieved pivots]; only the hot columns update the scores
        (stac/stac_voxel.py:208-267)."""
        slot = self._to_slot(layer_idx)
        T_main = self._offset_hot[slot]
        T_ret = self._offset_retrieval[slot]
        k_ret = v_ret = b_ret = None
        if T_ret > 0:
            k_ret = self.key_cache_retrieval[slot]
            v_ret = self.value_cache_retrieval[slot]
            b_ret = self._bias_retrieval[slot]
        out, colsum = self._attend(query_states, slot, k_ret, v_ret, b_ret, T_ret, want_colsum=True,
                                   subsample_ratio=self.subsample_ratio)
        self._last_query_offset[slot] = query_states.shape[1]
        self._update_scores_dev(colsum, colsum.stride(0), T_main, slot)
        if T_ret > 0:
            self._scores_retrieval[slot] = colsum[:, T_main:T_main + T_ret]
        return out

    # ------------------------------------------------------------------ positions
    def _search_recent_neighbors(self, slot_idx=0, dist_thres=0.1):
        """Voxels around the most recent tokens (stac/stac_voxel.py:294-323)."""
        import math
        TV = self._offset_voxel[slot_idx]
        R = min(self.recent_token_size, TV)
        if R == 0:
            self._recent_voxel_ids = None
            return
        if R < self.recent_token_size:
            self._recent_voxel_ids = self._vm.neighbor_ids(None, 0, all_ids=True)
            return
        tokens = self._token_voxel_indices[slot_idx, 0, TV - R:TV]
        cells = max(1, int(math.ceil(dist_thres / self._voxel_size_f)))
        self._recent_voxel_ids = self._vm.neighbor_ids(tokens, cells)

    @torch.no_grad()
    def append_positions(self, new_positions: torch.Tensor, new_pos_mask: torch.Tensor):
        """new_positions [T_new,3] fp32 world points, new_pos_mask [T_new] bool.  After append_kv
        of every layer, before prune_kv (stac/stac_voxel.py:326-365)."""
        T_new = new_positions.shape[0]
        if T_new == 0:
            return
        with self._stage("voxel_upsert"):
            ids = self._vm.upsert_points(new_positions, new_pos_mask)
        old_VT = self._offset_voxel[0]
        total = old_VT + T_new
        assert all(o == total for o in self._offset_hot), (
            f"[STACVoxelKV] size mismatch: hot_T={self._offset_hot} vs voxel_written={total}; "
            f"ensure append_kv -> append_positions")
        self._token_voxel_indices[:, :, old_VT:total].copy_(
            ids.view(1, 1, -1).expand(self._L_eff, self.num_heads, -1))
        self._offset_voxel = [total] * self._L_eff
        with self._stage("voxel_neighbors"):
            self._search_recent_neighbors(slot_idx=self._L_eff - 1, dist_thres=2 * self._voxel_size_f)

    @torch.no_grad()
    def append_pointmap(self, world_points: torch.Tensor, world_points_conf: torch.Tensor, patch_size: int,
                        conf_threshold: float = 1.0, special_tokens_size: int = 0):
        """get_pointmap + append_positions of the reference's streaming loop in one call
        (stream_session.py:213-256, aggregator.py:309-335): the chunk's world-point maps
        [S,H,W,3] / confidences [S,H,W] go straight to voxel ids without intermediate tensors on
        the host side.  Returns (pts3d [S,N,3], valid_mask [S,N]) like get_pointmap."""
        from .pointmap import pointmap_to_positions
        pts, mask = pointmap_to_positions(world_points, world_points_conf, patch_size, conf_threshold,
                                          special_tokens_size)
        self.append_positions(pts.view(-1, 3), mask.view(-1))
        return pts, mask

    def _clear_retrieval_cache(self, slot_idx: int):
        dev = self.device
        self._offset_retrieval[slot_idx] = 0
        self._scores_retrieval[slot_idx] = torch.zeros(self.num_heads, 0, device=dev, dtype=torch.float32)
        self.key_cache_retrieval[slot_idx] = torch.empty(self.num_heads, 0, self.head_dim, device=dev,
                                                         dtype=self.dtype)
        self.value_cache_retrieval[slot_idx] = torch.empty(self.num_heads, 0, self.head_dim, device=dev,
                                                           dtype=self.dtype)

    # ------------------------------------------------------------------ prune + eviction
    @torch.no_grad()
    def _apply_keep_and_compact_parallel(self, keep_idx_lh: torch.Tensor, drop_idx_lh: torch.Tensor = None):
        """Evicted tokens go to the voxel memory, then the cache is compacted
        (stac/stac_voxel.py:409-419)."""
        with self._stage("merge"):
            self._pool_drops_vectorized_parallel(keep_idx_lh, drop_idx_lh)
        with self._stage("compact"):
            self._compact(keep_idx_lh, vx=self._vx)
        self._token_voxel_indices = self._vx[self._cur]
        self._offset_voxel = [keep_idx_lh.shape[-1]] * self._L_eff

    def _pool_drops_vectorized_parallel(self, keep_idx_lh: torch.Tensor, drop_idx_lh: torch.Tensor):
        """stac/stac_voxel.py:421-488, with the dropped tokens read in place."""
        L, H, D = self._L_eff, self.num_heads, self.head_dim
        T, TV = self._offset_hot[0], self._offset_voxel[0]
        assert T == TV, (f"[STACVoxelKV] size mismatch T={T}, TV={TV};",
                         " must call: append_kv -> append_positions -> prune_kv")
        if T == 0:
            return
        T_d = T - keep_idx_lh.shape[-1]
        if T_d == 0:
            return
        Tb = self.reserved_buffer_token_size
        self._vstore.insert_evicted(self.key_cache_hot.view(L * H, Tb, D), self.value_cache_hot.view(L * H, Tb, D),
                                    self._scores_hot.view(L * H, Tb), self._token_voxel_indices.view(L * H, Tb),
                                    drop_idx_lh.view(L * H, T_d), T_d, self._vm.voxel_num_bound(),
                                    voxel_count_dev=self._vm._n_dev)

    # ------------------------------------------------------------------ retrieval
    def retrieve_kv(self, layer_idx, **kwargs):
        if self._to_slot(layer_idx) == 0:
            return self.retrieve_kv_parallel(**kwargs)
        return 0, 0

    @torch.no_grad()
    def retrieve_kv_parallel(self, **kwargs) -> Tuple[int, int]:
        """stac/stac_voxel.py:665-762: one retrieval for all layers; layer l then sees rows
        [l*H, (l+1)*H) of the result as views."""
        L, H = self._L_eff, self.num_heads
        voxel_ids = kwargs.get("voxel_ids", None)
        R = self.retrieval_token_size
        if voxel_ids is None:
            if self._vm.voxel_num_bound() == 0:
                for s in range(L):
                    self._clear_retrieval_cache(s)
                return 0, 0
            if self._recent_voxel_ids is None:
                return 0, 0
            ids, count = self._recent_voxel_ids
            if R <= 0:
                # unbounded mode: the output width depends on the data (one host read of the count)
                n = int(count.item())
                K, V, M, B = self._vstore.retrieve(voxel_ids=ids[:n], return_buf=kwargs.get("return_buf", False),
                                                   retrieve_size=R)
            else:
                with self._stage("retrieve"):
                    K, V, M, B = self._vstore.retrieve_device(ids, count, R)
        else:
            K, V, M, B = self._vstore.retrieve(voxel_ids=voxel_ids, return_buf=kwargs.get("return_buf", False),
                                               retrieve_size=R)
        self._ret = (K, V, M, B)
        Tm = K.shape[1] if R < 0 else min(K.shape[1], R)
        for s in range(L):
            self._clear_retrieval_cache(s)
            if Tm == 0:
                continue
            self.key_cache_retrieval[s] = K[s * H:(s + 1) * H, :Tm]
            self.value_cache_retrieval[s] = V[s * H:(s + 1) * H, :Tm]
            self._bias_retrieval[s] = B[s * H:(s + 1) * H, :Tm]
            self._offset_retrieval[s] = Tm
        return 0, 0

    # ------------------------------------------------------------------ public API
    def get_voxel_info(self) -> Dict[str, torch.Tensor]:
        return self._vm.get_voxel_info()

    def get_merger_info(self) -> Dict[str, torch.Tensor]:
        return self._vstore.info()

    def get_retrieval_size(self) -> List[int]:
        return self._offset_retrieval.copy()

    def get_memory_usage(self) -> Tuple[float, float]:
        usage_hot, alloc_hot = super().get_memory_usage()
        eb = torch.finfo(self.dtype).bits // 8
        ret = sum(self.num_heads * TR * self.head_dim * 2 * eb for TR in self._offset_retrieval) / (1024.0 ** 2)
        return usage_hot + ret, alloc_hot + ret

    def get_memory_voxel(self) -> Tuple[float, float]:
        st = self._vstore.memory()
        return (st["buffer_used_mem"] + st["pivot_used_mem"], st["buffer_alloc_mem"] + st["pivot_alloc_mem"])

    def get_memory_details(self) -> Dict[str, float]:
        """Same keys as stac/stac_voxel.py:854-952 (all in MB)."""
        H, D = self.num_heads, self.head_dim
        kvb = 2 * D * (torch.finfo(self.dtype).bits // 8)
        mb = 1024.0 ** 2
        pinned = window = hh = spatial = t_use = t_alloc = 0.0
        for l in range(self._L_eff):
            T_live = self._offset_hot[l]
            pc = min(len(self._pinned_token_index), T_live)
            rc = min(self.recent_token_size, T_live)
            hc = min(self.hh_token_size, max(0, T_live - pc - rc))
            pinned += H * pc * kvb / mb
            window += H * rc * kvb / mb
            hh += H * hc * kvb / mb
            spatial += H * self._offset_retrieval[l] * kvb / mb
            t_use += H * T_live * kvb / mb
            t_alloc += H * self.reserved_buffer_token_size * kvb / mb
        vs = self._vstore.memory() if self._vstore is not None else {}
        bu, ba = vs.get("buffer_used_mem", 0.0), vs.get("buffer_alloc_mem", 0.0)
        pu, pa = vs.get("pivot_used_mem", 0.0), vs.get("pivot_alloc_mem", 0.0)
        return {"pinned_memory": pinned, "window_memory": window, "heavy_hitters_memory": hh,
                "spatial_cache_usage": spatial, "spatial_cache_alloc": pu + bu,
                "voxel_buffer_usage": bu, "voxel_buffer_alloc": ba, "voxel_pivot_usage": pu,
                "voxel_pivot_alloc": pa, "temporal_cache_usage": t_use, "temporal_cache_alloc": t_alloc,
                "total_usage": t_use + spatial + bu + pu, "total_alloc": t_alloc + spatial + ba + pa}
