"""H2O heavy-hitter KV manager behind the reference's ``HeavyHittersKV`` interface
(stac/h2o.py:22-570).  Attention emits per-key softmax column sums which feed a decayed score
per cached token; pruning keeps pinned + recent + the top-scoring older tokens per (layer, head).
"""

import logging
import warnings
from typing import Optional

import torch

from .. import _lib
from .._lib import check, ptr, stream_ptr
from .kv_manager import KVManager

logger = logging.getLogger(__name__)


class HeavyHittersKV(KVManager):
    def __init__(self, *args, hh_size: int = 0, temperature: float = 1.0, attn_backend: str = "cuda",
                 subsample_ratio: float = 1.0, **kwargs):
        super().__init__(*args, **kwargs)
        self.attn_backend = str(attn_backend).strip().lower()
        if self.attn_backend not in ("cuda", "triton"):
            raise ValueError(f"attn_backend must be 'cuda' or 'triton', got '{attn_backend}'.")
        # both names select the one sm_100a kernel; the row sub-sampling rule follows the
        # reference's CUDA backend (exact at ratio 1)
        self.subsample_ratio = float(subsample_ratio)
        if not (0.0 < self.subsample_ratio <= 1.0):
            raise ValueError(f"subsample_ratio must be in (0, 1], got {self.subsample_ratio}.")
        self.use_attn_cuda = True
        self.hh_size = int(hh_size)
        self.cache_size = self.hh_size + self.recent_size
        self.hot_size = self.cache_size + self.pinned_size
        if self.reserved_buffer_size <= self.hot_size:
            warnings.warn(f"Warning: buffer_size {self.reserved_buffer_size} is smaller than "
                          f"hh_size+recent_size+pinned ({self.hot_size}). This may lead to no pruning.")
            self.reserved_buffer_size = self.hot_size + 1
            self.reserved_buffer_token_size = int(self.reserved_buffer_size * self.token_per_f)
        self.temperature = float(temperature)
        assert self.hh_size >= 0, "hh_size must be non-negative."
        assert self.temperature > 0, "temperature must be positive."
        self.hh_token_size = int(self.hh_size * self.token_per_f)
        self.cache_token_size = int(self.cache_size * self.token_per_f)
        self.hot_token_size = int(self.hot_size * self.token_per_f)
        self._scores_hot = None
        self._scores_hot_count = None
        self._last_score_offset = None
        self._last_query_offset = None

    # ------------------------------------------------------------------ core
    def reset(self):
        super().reset()
        L, H, T = self._L_eff, self.num_heads, self.reserved_buffer_token_size
        dev = self.device
        self._sc = [torch.zeros((L, H, T), dtype=torch.float32, device=dev) for _ in range(2)]
        self._cn = [torch.zeros((L, H, T), dtype=torch.float32, device=dev) for _ in range(2)]
        self._bind_scores()
        self._last_score_offset = [0] * L
        self._last_query_offset = [0] * L

    def state_dict(self):
        sd = super().state_dict()
        T = max(self._offset_hot)
        sd.update(scores=self._scores_hot[:, :, :T].cpu().clone(), counts=self._scores_hot_count[:, :, :T].cpu().clone(),
                  last_score_offset=list(self._last_score_offset), last_query_offset=list(self._last_query_offset))
        return sd

    def load_state_dict(self, sd):
        super().load_state_dict(sd)
        T = sd["scores"].shape[2]
        self._scores_hot[:, :, :T].copy_(sd["scores"])
        self._scores_hot_count[:, :, :T].copy_(sd["counts"])
        self._last_score_offset = list(sd["last_score_offset"])
        self._last_query_offset = list(sd["last_query_offset"])

    def _bind_scores(self):
        self._scores_hot = self._sc[self._cur]
        self._scores_hot_count = self._cn[self._cur]

    def free(self):
        self._scores_hot = self._scores_hot_count = None
        self._sc = self._cn = None
        self._last_score_offset = None
        self._last_query_offset = None
        super().free()

    @torch.no_grad()
    def decode_sparse_attn(self, query_states: torch.Tensor, layer_idx: int) -> torch.Tensor:
        """query_states [B, Tq, H, D] -> [B, Tq, H, D]; updates the hot scores (stac/h2o.py:139-174)."""
        slot = self._to_slot(layer_idx)
        out, colsum = self._attend(query_states, slot, want_colsum=True, subsample_ratio=self.subsample_ratio)
        self._last_query_offset[slot] = query_states.shape[1]
        self._update_scores_dev(colsum, colsum.stride(0), self._offset_hot[slot], slot)
        return out

    def _update_scores_dev(self, colsum, head_stride, T_live, slot):
        old_T = self._last_score_offset[slot]
        assert T_live <= self._offset_hot[slot], f"T_live({T_live}) > allocated({self._offset_hot[slot]})"
        Tb = self.reserved_buffer_token_size
        check(_lib.lib().stac_scores_update(ptr(colsum), head_stride, ptr(self._scores_hot[slot]),
                                            ptr(self._scores_hot_count[slot]), Tb, self.num_heads, T_live,
                                            old_T, self._last_query_offset[slot], self.temperature,
                                            stream_ptr()), "stac_scores_update")
        self._last_score_offset[slot] = T_live

    def _update_scores(self, scores: Optional[torch.Tensor] = None, slot_idx: int = 0):
        """scores [B, H, 1, T_live], already summed over the query rows (stac/h2o.py:177-216)."""
        if scores is None:
            return
        assert 0 <= slot_idx < self._L_eff, "Invalid slot_idx in _update_scores()."
        s = scores.sum(dim=(0, 2)).to(device=self.device, dtype=torch.float32).contiguous()
        H, T_live = s.shape
        assert H == self.num_heads, "Head mismatch in _update_scores"
        self._update_scores_dev(s, s.stride(0), T_live, slot_idx)

    # ------------------------------------------------------------------ prune
    def prune_kv(self):
        self._parallel_prune_kv()

    @torch.no_grad()
    def _parallel_prune_kv(self):
        """stac/h2o.py:244-354: keep = sort(pinned U recent U per-(layer, head) top-k of the rest)."""
        L, H = self._L_eff, self.num_heads
        if L == 0:
            return
        if any(o <= 0 for o in self._offset_hot):
            raise RuntimeError("Parallel prune failed: some slots are empty.")
        T = int(self._offset_hot[0])
        if any(o != T for o in self._offset_hot):
            raise RuntimeError(f"Parallel prune failed: slots have different live lengths: {self._offset_hot}.")
        if T <= max(self.hot_token_size, self.recent_token_size):
            return
        _, n_base = self._base_mask(T)
        if n_base == 0:
            raise RuntimeError("Parallel prune failed: no base tokens.")
        if n_base == T:
            return
        k = min(self.hh_token_size, T - n_base)
        if n_base + k == T:
            return  # every token is kept: the reference's compaction would be the identity
        Tb = self.reserved_buffer_token_size
        with self._stage("h2o_select"):
            keep, drop = self._select(self._scores_hot, Tb, L * H, T, n_base + k)
        self._apply_keep_and_compact_parallel(keep, drop)

    @torch.no_grad()
    def _apply_keep_and_compact_parallel(self, keep_idx_lh: torch.Tensor, drop_idx_lh: torch.Tensor = None):
        """keep_idx_lh int32 [L*H, T'] ascending kept positions (stac/h2o.py:356-436)."""
        self._compact(keep_idx_lh)

    def _compact(self, keep, vx=None):
        L, H, Tb, D = self._L_eff, self.num_heads, self.reserved_buffer_token_size, self.head_dim
        keep = keep.reshape(L * H, -1)
        n_keep = keep.shape[1]
        src, dst = self._cur, 1 - self._cur
        vs, vd = (None, None) if vx is None else (vx[src], vx[dst])
        check(_lib.lib().stac_compact(ptr(keep), L * H, n_keep, Tb, D, 2,
                                      ptr(self._kv[src][0]), ptr(self._kv[src][1]),
                                      ptr(self._kv[dst][0]), ptr(self._kv[dst][1]),
                                      ptr(self._ti[src]), ptr(self._ti[dst]),
                                      ptr(self._sc[src]), ptr(self._sc[dst]),
                                      ptr(self._cn[src]), ptr(self._cn[dst]), ptr(vs), ptr(vd),
                                      stream_ptr()), "stac_compact")
        self._cur = dst
        self._bind()
        self._bind_scores()
        self._offset_hot = [n_keep] * L
        self._last_score_offset = [min(x, n_keep) for x in self._last_score_offset]

    def get_scores(self) -> torch.Tensor:
        return self._scores_hot
