"""Sliding-window KV manager behind the reference's ``KVManager`` interface
(stac/kv_manager.py:13-530): a pre-allocated hot cache [L, H, T_buf, D] with token indices,
recent + pinned pruning with gather-compaction.

Differences that do not change results: the cache is double-buffered so compaction is a pure
gather into the second buffer (the attributes ``key_cache_hot`` / ``value_cache_hot`` always
name the live one); attention reads the [H, T, D] cache in place.  The CPU spill of buffers
longer than ``gpu_limit`` frames (stac/kv_manager.py:244-283) keeps the reference's rule (the
oldest tokens of an append that does not fit go to the host buffer, which only ever grows and
raises when full) with pinned host memory and stream-ordered copies; plain attention then reads
the spilled tokens as a second key segment from a device staging buffer.
"""

import gc
import logging
import warnings
from typing import List, Optional, Tuple, Union

import numpy as np
import torch

from .. import _lib, ops
from .._lib import check, ptr, stream_ptr

logger = logging.getLogger(__name__)


class _Stage:
    """Brackets one stage of the path with CUDA events when the manager has a trace sink
    (``manager.stage_trace = []``); does nothing otherwise.  The sink receives
    (stage name, start event, end event); nothing is synchronised here."""

    __slots__ = ("sink", "name", "e0")

    def __init__(self, sink, name):
        self.sink, self.name, self.e0 = sink, name, None

    def __enter__(self):
        if self.sink is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if self.sink is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.sink.append((self.name, self.e0, e1))
        return False


class KVManager:
    def __init__(self, num_layers: int, num_heads: int, head_dim: int, token_per_frame: int,
                 register_layers: Optional[List[int]] = None, chunk_size: int = 1, buffer_size: int = 8,
                 recent_size: int = 1, pinned_idx: Optional[List[int]] = None,
                 dtype: torch.dtype = torch.float16, device: Optional[torch.device] = None,
                 debug: bool = False, gpu_limit: int = 250, **kwargs):
        self.num_layers = int(num_layers)
        self.num_heads = int(num_heads)
        self.head_dim = int(head_dim)
        self.token_per_f = int(token_per_frame)
        self.reserved_buffer_size = int(buffer_size)
        if register_layers is None:
            managed = list(range(self.num_layers))
        else:
            managed = sorted({l for l in register_layers if 0 <= l < self.num_layers})
        if len(managed) == 0:
            raise ValueError("register_layers is empty after filtering valid indices.")
        self._managed_layers: List[int] = managed
        self._L_eff = len(managed)
        self._layer2slot = [-1] * self.num_layers
        for s, l in enumerate(managed):
            self._layer2slot[l] = s
        self.recent_size = int(recent_size)
        self.cache_size = self.recent_size
        pinned = [int(i) for i in (pinned_idx or [])]
        self.pinned_size = len(pinned)
        self.chunk_size = int(chunk_size)
        self.hot_size = self.cache_size + self.pinned_size
        if self.reserved_buffer_size < self.hot_size + self.chunk_size:
            warnings.warn(f"Warning: buffer_size {self.reserved_buffer_size} is smaller than "
                          f"hh_size+recent_size+pinned ({self.hot_size}). This may lead to no pruning.")
            self.reserved_buffer_size = self.hot_size + self.chunk_size
        self.reserved_buffer_size_cpu = max(self.reserved_buffer_size - gpu_limit, 0)
        self.reserved_buffer_size = min(self.reserved_buffer_size, gpu_limit)
        assert self.token_per_f > 0, "token_per_frame must be positive."
        assert self.recent_size >= 0, "recent_size and hh_size must be non-negative."
        assert self.cache_size > 0, "At least one of hh_size, recent_size, pinned_idx must be non-zero."
        self.recent_token_size = int(self.recent_size * self.token_per_f)
        self.cache_token_size = int(self.cache_size * self.token_per_f)
        self.reserved_buffer_token_size = int(self.reserved_buffer_size * self.token_per_f)
        self.reserved_buffer_token_size_cpu = int(self.reserved_buffer_size_cpu * self.token_per_f)
        self.hot_token_size = int(self.hot_size * self.token_per_f)
        self.chunk_token_size = int(self.chunk_size * self.token_per_f)
        tok = []
        for idx in pinned:
            if idx < 0:
                continue
            tok.extend(range(idx * self.token_per_f, (idx + 1) * self.token_per_f))
        self._pinned_token_index = torch.tensor(tok, dtype=torch.long)
        # The kernels compute and store in bfloat16.  float16 (the bare default of the reference's
        # StreamSession.register_kv_mgr, stream_session.py:580) is accepted for drop-in use: keys,
        # values and queries are converted at this boundary and outputs come back as float16.
        self.io_dtype = dtype
        if dtype == torch.float16:
            import warnings
            warnings.warn("stac_b200: dtype=float16 requested; the sm_100a kernels compute in bfloat16, tensors are "
                          "converted at the manager boundary", stacklevel=2)
            dtype = torch.bfloat16
        if dtype not in (torch.bfloat16,):
            raise ValueError("the sm_100a path computes in bfloat16; pass dtype=torch.bfloat16 (float16 is converted)")
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else torch.device("cuda")
        if self.device.type != "cuda":
            raise _lib.StacError("stac_b200 has no CPU path: a CUDA device is required")
        self.debug = debug
        self.key_cache_hot = None
        self.value_cache_hot = None
        self._token_indices_hot = None
        self._offset_hot = None
        self.use_cpu = False
        self._status = None
        self._base_cache = {}
        self._rope_rows = {}         # query length -> rows of the rotary tables (largest position + 1)
        self.stage_trace = None      # set to a list to collect (stage, start event, end event)

    def _stage(self, name):
        return _Stage(self.stage_trace, name)

    # ------------------------------------------------------------------ utilities
    def is_managed(self, layer_idx: int) -> bool:
        return self._layer2slot[layer_idx] >= 0

    def _to_slot(self, layer_idx: int, *, strict: bool = True) -> int:
        s = self._layer2slot[layer_idx]
        if s < 0 and strict:
            raise ValueError(f"Layer {layer_idx} is not managed by HeavyHittersKV.")
        return s

    def _layers_to_slots(self, layers: Union[List[int], torch.Tensor]) -> torch.Tensor:
        if isinstance(layers, torch.Tensor):
            layers = layers.tolist()
        return torch.tensor([self._layer2slot[l] for l in layers if self._layer2slot[l] >= 0],
                            dtype=torch.long, device=self.device)

    # ------------------------------------------------------------------ reset / free
    def _alloc_cache(self):
        L, H, T, D = self._L_eff, self.num_heads, self.reserved_buffer_token_size, self.head_dim
        dev = self.device
        self._kv = [(torch.empty(L, H, T, D, dtype=self.dtype, device=dev),
                     torch.empty(L, H, T, D, dtype=self.dtype, device=dev)) for _ in range(2)]
        self._ti = [torch.full((L, H, T), -1, dtype=torch.long, device=dev) for _ in range(2)]
        self._cur = 0
        self._bind()

    def _bind(self):
        self.key_cache_hot, self.value_cache_hot = self._kv[self._cur]
        self._token_indices_hot = self._ti[self._cur]

    def reset(self):
        self._processed_frames = 0
        self._status = ops.DeviceStatus(self.device)
        self._alloc_cache()
        self._offset_hot = [0] * self._L_eff
        self._offset_hot_cpu = [0] * self._L_eff
        self.use_cpu = False
        T_cpu = self.reserved_buffer_token_size_cpu
        self.key_cache_hot_cpu = self.value_cache_hot_cpu = None
        self._cpu_stage = None
        if T_cpu > 0:
            shape = (self._L_eff, self.num_heads, T_cpu, self.head_dim)
            self.key_cache_hot_cpu = torch.empty(shape, dtype=self.dtype).pin_memory()
            self.value_cache_hot_cpu = torch.empty(shape, dtype=self.dtype).pin_memory()

    def free(self):
        self._processed_frames = 0
        self.key_cache_hot = self.value_cache_hot = self._token_indices_hot = None
        self._kv = self._ti = None
        self._offset_hot = None
        self._offset_hot_cpu = None
        self.key_cache_hot_cpu = self.value_cache_hot_cpu = None
        self._cpu_stage = None
        gc.collect()
        torch.cuda.synchronize(self.device)
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        """Live contents of the hot cache (and of the host spill buffer) with their counters, on
        the CPU.  The reference has no checkpointing; a stream restored with load_state_dict
        continues with the same bits as the uninterrupted one."""
        T = max(self._offset_hot)
        Tc = max(self._offset_hot_cpu) if self.key_cache_hot_cpu is not None else 0
        cpu = lambda t: t.cpu().clone()
        return {
            "format": 1, "class": type(self).__name__,
            "shape": [self._L_eff, self.num_heads, self.head_dim, self.token_per_f, self.reserved_buffer_token_size],
            "processed_frames": int(self._processed_frames), "offset_hot": list(self._offset_hot),
            "key": cpu(self.key_cache_hot[:, :, :T]), "value": cpu(self.value_cache_hot[:, :, :T]),
            "token_idx": cpu(self._token_indices_hot[:, :, :T]),
            "use_cpu": bool(self.use_cpu), "offset_hot_cpu": list(self._offset_hot_cpu),
            "key_cpu": self.key_cache_hot_cpu[:, :, :Tc].clone() if Tc else None,
            "value_cpu": self.value_cache_hot_cpu[:, :, :Tc].clone() if Tc else None,
        }

    def load_state_dict(self, sd):
        """Into a manager constructed with the same arguments (checked); resets it first."""
        if sd.get("format") != 1 or sd.get("class") != type(self).__name__:
            raise ValueError(f"state of {sd.get('class')} (format {sd.get('format')}) does not fit {type(self).__name__}")
        shape = [self._L_eff, self.num_heads, self.head_dim, self.token_per_f, self.reserved_buffer_token_size]
        if list(sd["shape"]) != shape:
            raise ValueError(f"state was saved with [layers, heads, head_dim, tokens/frame, buffer tokens] = "
                             f"{list(sd['shape'])}, this manager has {shape}")
        self.reset()
        T = sd["key"].shape[2]
        self.key_cache_hot[:, :, :T].copy_(sd["key"])
        self.value_cache_hot[:, :, :T].copy_(sd["value"])
        self._token_indices_hot[:, :, :T].copy_(sd["token_idx"])
        self._offset_hot = list(sd["offset_hot"])
        self._processed_frames = int(sd["processed_frames"])
        self.use_cpu = bool(sd["use_cpu"])
        self._offset_hot_cpu = list(sd["offset_hot_cpu"])
        if sd["key_cpu"] is not None:
            Tc = sd["key_cpu"].shape[2]
            self.key_cache_hot_cpu[:, :, :Tc].copy_(sd["key_cpu"])
            self.value_cache_hot_cpu[:, :, :Tc].copy_(sd["value_cpu"])

    # ------------------------------------------------------------------ append
    def append_kv(self, key_states, value_states, layer_idx: int):
        """key_states, value_states: [B, H, T_new, D] with B == 1."""
        B, H, new_T, D = key_states.shape
        assert H == self.num_heads and D == self.head_dim, "Incompatible head or head_dim."
        assert B == 1, "Batch size > 1 not supported in append_kv()."
        assert new_T % self.token_per_f == 0, "T_new must be a multiple of token_per_frame in append_kv()."
        slot = self._to_slot(layer_idx, strict=True)
        old_T = self._offset_hot[slot]
        k, v = key_states[0], value_states[0]
        if k.dtype != self.dtype or v.dtype != self.dtype or not k.is_cuda:
            k, v = k.to(self.device, self.dtype), v.to(self.device, self.dtype)
        # the GPU buffer takes the LAST tokens that fit, the host buffer the first ones
        # (stac/kv_manager.py:244-283); token ids are kept for the GPU part only
        to_gpu = min(new_T, max(self.reserved_buffer_token_size - old_T, 0))
        to_cpu = new_T - to_gpu
        if to_cpu > 0:
            warnings.warn(f"Exceeding GPU buffer token size {self.reserved_buffer_token_size} in append_kv(). "
                          f"{to_cpu} tokens will be stored on CPU.")
            self.use_cpu = True
            if self.reserved_buffer_token_size_cpu > 0:
                old_c = self._offset_hot_cpu[slot]
                if old_c + to_cpu > self.reserved_buffer_token_size_cpu:
                    raise RuntimeError("CPU buffer overflow in append_kv(). Increase gpu_limit or buffer_size.")
                self.key_cache_hot_cpu[slot, :, old_c:old_c + to_cpu].copy_(k[:, :to_cpu], non_blocking=True)
                self.value_cache_hot_cpu[slot, :, old_c:old_c + to_cpu].copy_(v[:, :to_cpu], non_blocking=True)
                self._offset_hot_cpu[slot] = old_c + to_cpu
        F_new = new_T // self.token_per_f
        first_id = self._processed_frames * self.token_per_f + to_cpu
        if slot == self._L_eff - 1:
            self._processed_frames += F_new
        if to_gpu == 0:
            return
        k, v = k[:, to_cpu:], v[:, to_cpu:]
        new_T = to_gpu
        if k.stride(2) != 1 or (k.stride(0) % 8) or (k.stride(1) % 8) or (k.data_ptr() % 16):
            k = k.contiguous()
        if v.stride(2) != 1 or (v.stride(0) % 8) or (v.stride(1) % 8) or (v.data_ptr() % 16):
            v = v.contiguous()
        F_new = new_T // self.token_per_f
        kc, vc, ti = self.key_cache_hot[slot], self.value_cache_hot[slot], self._token_indices_hot[slot]
        check(_lib.lib().stac_append_kv(ptr(k), ptr(v), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                                        ptr(kc), ptr(vc), kc.stride(0), ptr(ti), ti.stride(0), H, new_T, old_T,
                                        first_id, D, 2, stream_ptr()),
              "stac_append_kv")
        self._offset_hot[slot] = old_T + new_T

    @torch.no_grad()
    def append_qkv(self, qkv, layer_idx: int, *, q_norm=None, k_norm=None, rope=None, pos=None):
        """The attention layer's projection epilogue and append_kv in one kernel
        (causalvggt/layers/attention.py:119-128, :141): `qkv` is the output of the layer's QKV
        projection, [1, T, 3*H*D] (or [1, T, 3, H, D]) bf16; `q_norm` / `k_norm` are the layer's
        ``nn.LayerNorm(head_dim)`` modules (None or Identity: no normalisation); `rope` is its
        ``RotaryPositionEmbedding2D`` (its own frequency cache supplies the cos / sin values) with
        `pos` [1, T, 2] integer (y, x) positions, or None.  K and V go straight into the cache
        tail (no [B,H,T,D] copies are ever made); returns q [1, T, H, D] bf16, ready for
        decode_sparse_attn."""
        H, D = self.num_heads, self.head_dim
        if D != 64:
            raise ValueError("the fused epilogue supports head_dim 64")
        assert qkv.is_cuda and qkv.shape[0] == 1, "qkv: [1, T, 3*H*D] on the GPU"
        out_dtype = qkv.dtype
        if qkv.dtype != torch.bfloat16:
            assert qkv.dtype == self.io_dtype, "qkv must be bf16 (or the float16 the manager was created with)"
            qkv = qkv.to(torch.bfloat16)
        T_new = qkv.shape[1]
        x = qkv.reshape(T_new, 3 * H * D)
        if x.stride(1) != 1 or x.data_ptr() % 4:
            x = x.contiguous()
        assert T_new % self.token_per_f == 0, "T_new must be a multiple of token_per_frame in append_qkv()."
        slot = self._to_slot(layer_idx, strict=True)
        old_T = self._offset_hot[slot]
        if old_T + T_new > self.reserved_buffer_token_size:
            raise RuntimeError("the fused epilogue writes to the GPU buffer only; use append_kv when tokens spill to the host")

        def affine(mod):
            if mod is None or not hasattr(mod, "weight") or mod.weight is None:
                return None, None, 1e-5
            w = mod.weight.detach().to(self.device, torch.float32).contiguous()
            b = (mod.bias.detach().to(self.device, torch.float32).contiguous() if mod.bias is not None
                 else torch.zeros_like(w))
            return w, b, float(mod.eps)
        qw, qb, eps = affine(q_norm)
        kw, kb, eps_k = affine(k_norm)
        eps = eps if qw is not None else eps_k
        cos = sin = p64 = None
        n_pos = 0
        if rope is not None:
            assert pos is not None and pos.shape[-1] == 2 and pos.shape[-2] == T_new
            p64 = pos.reshape(T_new, 2).to(self.device, torch.int64).contiguous()
            n_pos = self._rope_rows.get(T_new)
            if n_pos is None:          # one host read per query length: positions repeat chunk after chunk
                n_pos = int(p64.max().item()) + 1
                self._rope_rows[T_new] = n_pos
            c32, s32 = rope._compute_frequency_components(D // 2, n_pos, self.device, torch.float32)
            cos, sin = c32[:, : D // 4].contiguous(), s32[:, : D // 4].contiguous()
        q_out = torch.empty((1, T_new, H, D), dtype=torch.bfloat16, device=self.device)
        kc, vc, ti = self.key_cache_hot[slot], self.value_cache_hot[slot], self._token_indices_hot[slot]
        first_id = self._processed_frames * self.token_per_f
        check(_lib.lib().stac_qkv_epilogue_append(
            ptr(x), x.stride(0), ptr(qw), ptr(qb), ptr(kw), ptr(kb), eps, ptr(p64), ptr(cos), ptr(sin), n_pos,
            ptr(q_out), q_out.stride(1), ptr(kc), ptr(vc), kc.stride(0), ptr(ti), ti.stride(0), H, T_new, old_T,
            first_id, stream_ptr()), "stac_qkv_epilogue_append")
        if slot == self._L_eff - 1:
            self._processed_frames += T_new // self.token_per_f
        self._offset_hot[slot] = old_T + T_new
        return q_out if out_dtype == torch.bfloat16 else q_out.to(out_dtype)

    @torch.no_grad()
    def prefill(self, query_states, key_states, value_states, layer_idx: int):
        """query/key/value [B, T, H, D] (stac/kv_manager.py:195-224)."""
        B, T, H, D = query_states.shape
        assert H == self.num_heads and D == self.head_dim and B == 1
        assert T % self.token_per_f == 0
        self.reset()
        slot = self._to_slot(layer_idx, strict=True)
        self.key_cache_hot[slot, :, :T, :].copy_(key_states[0].transpose(0, 1))
        self.value_cache_hot[slot, :, :T, :].copy_(value_states[0].transpose(0, 1))
        self._offset_hot[slot] = T
        out = self.decode_sparse_attn(query_states, layer_idx)
        F = T // self.token_per_f
        self._processed_frames = F
        self._token_indices_hot[slot, :, :T].copy_(torch.arange(T, device=self.device).expand(H, -1))
        return out

    # ------------------------------------------------------------------ attention
    def _attend(self, query_states, slot, k_ret=None, v_ret=None, bias_ret=None, T_ret=0,
                want_colsum=False, subsample_ratio=1.0):
        B, Tq, H, D = query_states.shape
        assert H == self.num_heads and D == self.head_dim, "Incompatible head or head_dim."
        assert B == 1, "Batch size > 1 not supported in decode_sparse_attn()."
        assert query_states.is_cuda, "decode_sparse_attn requires CUDA tensors"
        out_dtype = query_states.dtype
        if out_dtype != torch.bfloat16:
            assert out_dtype == self.io_dtype, "q must be bf16 (or the float16 the manager was created with)"
            query_states = query_states.to(torch.bfloat16)
        q = query_states[0]
        if q.stride(2) != 1 or q.stride(1) != D:
            q = q.contiguous()
        T_main = self._offset_hot[slot]
        out, _, colsum = ops.attn_colsum(q, self.key_cache_hot[slot], self.value_cache_hot[slot], T_main,
                                         k_ret, v_ret, bias_ret, T_ret, subsample_ratio=subsample_ratio,
                                         want_colsum=want_colsum, status=self._status)
        out = out.unsqueeze(0)
        return (out if out_dtype == torch.bfloat16 else out.to(out_dtype)), colsum

    @torch.no_grad()
    def decode_sparse_attn(self, query_states: torch.Tensor, layer_idx: int) -> torch.Tensor:
        """Plain attention over the hot cache and, once tokens were spilled, the host part as well
        (stac/kv_manager.py:311-360); query_states [B, Tq, H, D] -> [B, Tq, H, D]."""
        slot = self._to_slot(layer_idx, strict=True)
        T_cpu = self._offset_hot_cpu[slot] if self.use_cpu and self.key_cache_hot_cpu is not None else 0
        if T_cpu == 0:
            out, _ = self._attend(query_states, slot)
            return out
        # bring the spilled tokens back into a device staging buffer (stream-ordered copies from
        # pinned memory) and attend over them as a second key segment with zero bias
        if self._cpu_stage is None:
            shape = (self.num_heads, self.reserved_buffer_token_size_cpu, self.head_dim)
            self._cpu_stage = (torch.empty(shape, dtype=self.dtype, device=self.device),
                               torch.empty(shape, dtype=self.dtype, device=self.device),
                               torch.zeros(shape[:2], dtype=torch.float32, device=self.device))
        ks, vs, zero_bias = self._cpu_stage
        ks[:, :T_cpu].copy_(self.key_cache_hot_cpu[slot, :, :T_cpu], non_blocking=True)
        vs[:, :T_cpu].copy_(self.value_cache_hot_cpu[slot, :, :T_cpu], non_blocking=True)
        out, _ = self._attend(query_states, slot, ks, vs, zero_bias, T_cpu)
        return out

    # ------------------------------------------------------------------ prune
    def _base_mask(self, T):
        """uint8 [T] device mask of the always-kept positions (pinned < T and the recent tail),
        plus its size (stac/kv_manager.py:381-391, stac/h2o.py:279-295)."""
        hit = self._base_cache.get(T)
        if hit is None:
            m = np.zeros(T, np.uint8)
            m[T - min(self.recent_token_size, T):] = 1
            pinned = self._pinned_token_index.numpy()
            pinned = pinned[(pinned >= 0) & (pinned < T)]
            m[pinned] = 1
            hit = (torch.from_numpy(m).to(self.device), int(m.sum()))
            self._base_cache = {T: hit}
        return hit

    def _select(self, scores_rows, row_stride, n_rows, T, n_keep):
        base, _ = self._base_mask(T)
        keep = torch.empty((n_rows, n_keep), dtype=torch.int32, device=self.device)
        drop = torch.empty((n_rows, T - n_keep), dtype=torch.int32, device=self.device)
        check(_lib.lib().stac_h2o_select(ptr(scores_rows), row_stride, n_rows, ptr(base), T, n_keep,
                                         ptr(keep), ptr(drop), stream_ptr()), "stac_h2o_select")
        return keep, drop

    @torch.no_grad()
    def prune_kv(self):
        """Keep pinned + recent tokens, compact (stac/kv_manager.py:362-441), all layers at once."""
        L, H = self._L_eff, self.num_heads
        T = self._offset_hot[0]
        if T == 0 or any(o != T for o in self._offset_hot):
            if T == 0:
                return
            raise RuntimeError(f"prune_kv requires equal live lengths, got {self._offset_hot}")
        if T <= max(self.hot_token_size, self.recent_token_size):
            return
        _, n_base = self._base_mask(T)
        if n_base == T:
            return
        zeros = torch.zeros((L * H, T), dtype=torch.float32, device=self.device)
        keep, _ = self._select(zeros, T, L * H, T, n_base)
        self._compact(keep)

    def _compact(self, keep):
        """Gather-compaction into the idle buffers, then swap."""
        L, H, Tb, D = self._L_eff, self.num_heads, self.reserved_buffer_token_size, self.head_dim
        n_keep = keep.shape[1]
        src, dst = self._cur, 1 - self._cur
        zs = getattr(self, "_zero_meta", None)
        if zs is None:
            zs = [torch.zeros((L, H, Tb), dtype=torch.float32, device=self.device) for _ in range(2)]
            self._zero_meta = zs
        check(_lib.lib().stac_compact(ptr(keep), L * H, n_keep, Tb, D, 2,
                                      ptr(self._kv[src][0]), ptr(self._kv[src][1]),
                                      ptr(self._kv[dst][0]), ptr(self._kv[dst][1]),
                                      ptr(self._ti[src]), ptr(self._ti[dst]),
                                      ptr(zs[0]), ptr(zs[1]), ptr(zs[0]), ptr(zs[1]), None, None,
                                      stream_ptr()), "stac_compact")
        self._cur = dst
        self._bind()
        self._offset_hot = [n_keep] * L

    @torch.no_grad()
    def retrieve_kv(self, layer_idx: int, **kwargs) -> Tuple[int, int]:
        raise NotImplementedError("retrieve_kv() is not implemented for HeavyHittersKV.")

    @torch.no_grad()
    def append_positions(self, new_positions: torch.Tensor, new_pos_mask: torch.Tensor):
        raise NotImplementedError("append_positions() is not implemented for HeavyHittersKV.")

    # ------------------------------------------------------------------ public API
    def get_token_indices(self) -> torch.Tensor:
        return self._token_indices_hot.clone().cpu()

    def get_layers(self) -> List[int]:
        return self._managed_layers.copy()

    def get_kv(self):
        return self.key_cache_hot.clone().cpu(), self.value_cache_hot.clone().cpu()

    def get_offset(self) -> List[int]:
        return self._offset_hot.copy()

    def get_offset_cpu(self) -> List[int]:
        if getattr(self, "_offset_hot_cpu", None) is None:
            return [0] * self._L_eff
        return self._offset_hot_cpu.copy()

    def get_cpu_memory_usage(self) -> Tuple[float, float]:
        """(used MB, allocated MB) of the host part; zeros while nothing was spilled
        (stac/kv_manager.py:488-503)."""
        if not getattr(self, "use_cpu", False) or getattr(self, "_offset_hot_cpu", None) is None:
            return 0.0, 0.0
        eb = torch.finfo(self.dtype).bits // 8
        mb = 1024.0 ** 2
        usage = sum(2 * self.num_heads * T * self.head_dim * eb for T in self._offset_hot_cpu) / mb
        alloc = self._L_eff * 2 * self.reserved_buffer_token_size_cpu * self.num_heads * self.head_dim * eb / mb
        return usage, alloc

    def get_memory_usage(self) -> Tuple[float, float]:
        eb = torch.finfo(self.dtype).bits // 8
        mb = 1024.0 ** 2
        usage = sum(2 * self.num_heads * T * self.head_dim * eb for T in self._offset_hot) / mb
        alloc = self._L_eff * 2 * self.reserved_buffer_token_size * self.num_heads * self.head_dim * eb / mb
        return usage, alloc

    def get_memory_details(self) -> dict:
        used, alloc = self.get_memory_usage()
        return {"total_usage": used, "total_alloc": alloc, "temporal_cache_usage": used,
                "temporal_cache_alloc": alloc, "spatial_cache_usage": 0.0}

    def check_status(self):
        """Synchronise and raise if any kernel reported a device-side error."""
        if self._status is not None:
            self._status.raise_if_set(type(self).__name__)
