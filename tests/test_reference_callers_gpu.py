"""The managers of this library driven by the reference's OWN callers.

Needs ``oracle/_ref`` (``python oracle/make_ref.py /path/to/reference``: the reference's Python
sources, staged git-ignored); skipped with that reason otherwise.

* ``SparseAttention.forward(..., kv_manager=STACVoxelKV)`` (causalvggt/layers/attention.py:113-161)
  against the same module's plain softmax branch (``fused_attn=False``);
* ``CausalAggregator.register_kv_mgr / inference / update_kv_mgr_pos / retrieve_kv_mgr /
  prune_kv_mgr / get_kv_mgr_info`` (causalvggt/models/aggregator.py:159-335, :487-600) with this
  library's manager and with the reference's own (Triton attention, Python voxel path) on the
  same seeded stream;
* ``StreamSession.pipeline`` (stream_session.py:258-565), unchanged, in a child process where
  ``import stac`` resolves to this library.
"""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
needs_ref = pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "stream_session.py")),
                               reason="oracle/_ref not staged (python oracle/make_ref.py <reference checkout>)")


@pytest.fixture(scope="module")
def ref_modules():
    """Import the reference's causalvggt with ITS OWN stac package (from oracle/_ref)."""
    assert "stac" not in sys.modules or "_ref" in getattr(sys.modules["stac"], "__file__", "")
    sys.path.insert(0, REF)
    try:
        import logging
        logging.disable(logging.INFO)
        from causalvggt.layers.attention import SparseAttention
        from causalvggt.layers.rope import PositionGetter, RotaryPositionEmbedding2D
        from causalvggt.models.aggregator import CausalAggregator
        from stac.stac_voxel import STACVoxelKV as RefSTACVoxelKV
        yield dict(SparseAttention=SparseAttention, PositionGetter=PositionGetter,
                   Rope=RotaryPositionEmbedding2D, CausalAggregator=CausalAggregator,
                   RefSTACVoxelKV=RefSTACVoxelKV)
    finally:
        sys.path.remove(REF)


def _manager_kwargs(tpf, dev, **over):
    """What StreamSession.register_kv_mgr passes for the `stac` preset (stream_session.py:399-419, :572-612)."""
    kw = dict(chunk_size=2, recent_size=3, pinned_idx=[0], hh_size=1, persist_size=0, temperature=0.9,
              device=dev, dtype=torch.bfloat16, register_layers=None, window_size=3,
              token_per_frame=tpf, buffer_size=2 + 1 + 3 + 1,
              voxel_size=0.05, voxelize_layers=None, init_voxels=64, voxel_buf_cap=8, voxel_piv_cap=4,
              voxel_backend="python", sim_threshold=0.8, replace_threshold=0.8, score_threshold=0.2,
              slab_growth=1024, slab_cap=10000, seg_size=1, retrieval_size=1, allocator="segment",
              enable_alloc_cpu=False, gpu_threshold_gb=10.0, cold_frame_threshold=5,
              attn_backend="triton", subsample_ratio=1.0, return_buf=True, conf_threshold=1.0)
    kw.update(over)
    return kw


@needs_ref
def test_sparse_attention_forward_uses_the_manager(ref_modules):
    from stac_b200.stac import STACVoxelKV
    dev = torch.device("cuda:0")
    torch.manual_seed(3)
    dim, heads, ph, pw, special = 128, 2, 4, 5, 5
    tpf = ph * pw + special
    rope = ref_modules["Rope"](frequency=100)
    attn = ref_modules["SparseAttention"](dim=dim, num_heads=heads, qk_norm=True, rope=rope).to(dev, torch.bfloat16).eval()
    attn.set_layer_idx(0)
    pos = ref_modules["PositionGetter"]()(1, ph, pw, device=dev) + 1
    pos = torch.cat([torch.zeros(1, special, 2, device=dev, dtype=pos.dtype), pos], 1)      # one frame
    mgr = STACVoxelKV(num_layers=1, num_heads=heads, head_dim=dim // heads, **_manager_kwargs(tpf, dev))
    mgr.reset()
    frames = [2, 2, 2]
    xs = [torch.randn(1, f * tpf, dim, device=dev, dtype=torch.bfloat16) for f in frames]
    outs = []
    with torch.no_grad():
        for x, f in zip(xs, frames):
            outs.append(attn(x, pos=pos.repeat(1, f, 1), kv_manager=mgr))
        mgr.check_status()
        # the same module on its plain softmax branch sees all tokens at once: the rows of chunk c
        # attend to chunks 0..c in the manager, so compare with a run over exactly those tokens
        attn.fused_attn = False
        for c in range(len(frames)):
            x_all = torch.cat(xs[:c + 1], 1)
            p_all = pos.repeat(1, sum(frames[:c + 1]), 1)
            ref = attn(x_all, pos=p_all)[:, -frames[c] * tpf:]
            err = (outs[c].float() - ref.float()).abs().max().item()
            assert err <= 3e-2, (c, err)
    assert mgr.get_offset() == [sum(frames) * tpf]


def _drive(agg, steps, S, Hpx, Wpx, dev, seed, retrieve_from=4):
    """The per-chunk calls of StreamSession.pipeline's STAC branch (stream_session.py:451-493)
    on a CausalAggregator, with seeded frames and seeded (injected) point maps."""
    rs = np.random.RandomState(seed)
    tpf = (Hpx // 14) * (Wpx // 14) + agg.patch_start_idx
    trace = []
    for step in range(steps):
        imgs = torch.from_numpy(rs.rand(1, S, 3, Hpx, Wpx).astype(np.float32)).to(dev)
        with torch.no_grad(), torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
            out = agg.inference(imgs, mode="full", is_anchor_exist=(step == 0))
        pts = torch.zeros(S, tpf, 3)
        mask = torch.zeros(S, tpf, dtype=torch.bool)
        npatch = tpf - agg.patch_start_idx
        base = rs.rand(S, npatch, 3).astype(np.float32) * np.float32(0.4)
        base[..., 0] += np.float32(0.03 * step)
        pts[:, agg.patch_start_idx:] = torch.from_numpy(base)
        mask[:, agg.patch_start_idx:] = torch.from_numpy(rs.rand(S, npatch) < 0.9)
        agg.update_kv_mgr_pos(pts.to(dev), mask.to(dev), timing=True)
        if step >= retrieve_from:
            agg.retrieve_kv_mgr(timing=True, verbose=False, dist_thres=0.1, return_buf=True)
        agg.prune_kv_mgr(timing=True)
        info = agg.get_kv_mgr_info()
        trace.append(dict(tokens=out["output_list"][4].float().cpu(), offset=list(info["kvcache_size"]),
                          token_indices=info["token_indices"].copy(), retrieval=list(info["retrieval_size"]),
                          merger=agg.kv_manager.get_merger_info(), mem=agg.kv_manager.get_memory_details()))
    return trace


@needs_ref
def test_aggregator_hooks_match_the_reference_manager(ref_modules):
    from stac_b200.stac import STACVoxelKV
    dev = torch.device("cuda:0")
    Hpx, Wpx, S, steps = 56, 70, 2, 9
    tpf = (Hpx // 14) * (Wpx // 14) + 5

    def build(manager):
        torch.manual_seed(7)
        agg = ref_modules["CausalAggregator"](img_size=70, patch_size=14, embed_dim=128, depth=5, num_heads=2,
                                              patch_embed="conv").to(dev).eval()
        agg.register_kv_mgr(kv_manager=manager, **_manager_kwargs(tpf, dev))
        return agg

    ours = _drive(build(STACVoxelKV), steps, S, Hpx, Wpx, dev, seed=11)
    theirs = _drive(build(ref_modules["RefSTACVoxelKV"]), steps, S, Hpx, Wpx, dev, seed=11)
    saw_retrieval = False
    for a, b in zip(ours, theirs):
        assert a["offset"] == b["offset"]
        assert a["retrieval"] == b["retrieval"]
        saw_retrieval |= any(r > 0 for r in a["retrieval"])
        # same kept tokens except where two scores are closer than the rounding of the two attention kernels
        same = (a["token_indices"] == b["token_indices"]).mean()
        assert same >= 0.97, same
        scale = b["tokens"].abs().mean().item()
        assert (a["tokens"] - b["tokens"]).abs().mean().item() <= 0.03 * scale
        assert set(b["mem"].keys()) <= set(a["mem"].keys())
        for key in ("used_voxels", "token_count"):
            assert int(a["merger"][key]) == int(b["merger"][key]), key
        # pool fill depends on the kept sets above; allow the same slack
        for key in ("pivot_pool_used", "buffer_pool_used"):
            assert abs(int(a["merger"][key]) - int(b["merger"][key])) <= 0.05 * max(int(b["merger"][key]), 20), key
    assert saw_retrieval


@needs_ref
def test_stream_session_pipeline_runs_unchanged():
    cmd = [sys.executable, os.path.join(ROOT, "tests", "stream_session_run.py"), "--manager", "stac_b200",
           "--model", "tiny", "--frames", "32"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["manager_module"].startswith("stac_b200/stac/"), out["manager_module"]
    assert out["processed_frames"] == 32 and out["finite"]
    for key in ("temporal_cache_usage", "spatial_cache_usage", "voxel_buffer_usage", "voxel_pivot_usage",
                "voxel_buffer_alloc", "voxel_pivot_alloc", "total_usage"):
        assert key in out["memory_keys"], key
    assert out["memory_mb"]["voxel_buffer_usage"] + out["memory_mb"]["voxel_pivot_usage"] > 0, \
        "no token reached the voxel memory"
    for stage in ("aggregator_infer_time", "kv_position_time", "kv_retrieval_time", "kv_evict_merge_time"):
        assert stage in out["stage_ms_per_frame"], stage


@needs_ref
def test_fused_qkv_epilogue_matches_the_reference_layer(ref_modules):
    """append_qkv (LayerNorm of q and k, 2-D rotary embedding, bf16 rounding, K/V and token ids
    written into the cache tail in one kernel) against the lines of the reference's
    SparseAttention.forward that it replaces (causalvggt/layers/attention.py:117-128, :141), run
    under bf16 autocast as main.py runs them."""
    from stac_b200.stac import STACVoxelKV
    dev = torch.device("cuda:0")
    torch.manual_seed(9)
    dim, heads, ph, pw, special = 256, 4, 5, 6, 5
    tpf = ph * pw + special
    rope = ref_modules["Rope"](frequency=100)
    attn = ref_modules["SparseAttention"](dim=dim, num_heads=heads, qk_norm=True, rope=rope).to(dev).eval()
    with torch.no_grad():        # non-trivial affine parameters
        for ln in (attn.q_norm, attn.k_norm):
            ln.weight.copy_(1 + 0.2 * torch.randn_like(ln.weight))
            ln.bias.copy_(0.1 * torch.randn_like(ln.bias))
    attn.set_layer_idx(0)
    pos1 = ref_modules["PositionGetter"]()(1, ph, pw, device=dev) + 1
    pos1 = torch.cat([torch.zeros(1, special, 2, device=dev, dtype=pos1.dtype), pos1], 1)
    mgr = STACVoxelKV(num_layers=1, num_heads=heads, head_dim=dim // heads, **_manager_kwargs(tpf, dev))
    mgr.reset()
    done = 0
    for frames in (2, 1):
        N = frames * tpf
        x = torch.randn(1, N, dim, device=dev) * 2
        pos = pos1.repeat(1, frames, 1)
        with torch.no_grad(), torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
            qkv = attn.qkv(x)                                                    # the projection itself
            r = qkv.reshape(1, N, 3, heads, dim // heads).permute(2, 0, 3, 1, 4)
            q, k, v = r.unbind(0)
            q, k = attn.q_norm(q), attn.k_norm(k)
            q = attn.rope(q, pos).type_as(v)
            k = attn.rope(k, pos).type_as(v)
        q_ours = mgr.append_qkv(qkv, 0, q_norm=attn.q_norm, k_norm=attn.k_norm, rope=attn.rope, pos=pos)
        torch.cuda.synchronize()

        def ulps(a, b):          # distance in bf16 steps of the larger magnitude
            a, b = a.float(), b.float()
            return ((a - b).abs() / (torch.maximum(a.abs(), b.abs()).clamp_min(1e-3) * 2 ** -7)).max().item()
        assert ulps(q_ours[0], q[0].transpose(0, 1)) <= 1.01
        assert ulps(mgr.key_cache_hot[0][:, done:done + N], k[0]) <= 1.01
        assert torch.equal(mgr.value_cache_hot[0][:, done:done + N], v[0])
        want_ids = torch.arange(done, done + N, device=dev).expand(heads, -1)
        assert torch.equal(mgr._token_indices_hot[0][:, done:done + N], want_ids)
        done += N
    assert mgr.get_offset() == [done]
