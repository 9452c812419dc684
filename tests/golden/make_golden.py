"""Generate the golden fixtures in this directory by running the reference's own Python
path (CPU, ``voxel_backend="python"``, ``allocator="segment"``, ``seg_size=1``).

Usage (needs a checkout of the reference; not needed to run the tests):

    python tests/golden/make_golden.py /path/to/reference

Inputs are drawn from ``numpy.random.RandomState`` with the seeds in ``cases.py`` so the
tests can rebuild them without storing them; only the reference's outputs are saved.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def _import_reference(path):
    sys.path.insert(0, path)
    import torch  # noqa: F401
    from stac.merger import VoxelKVMerger
    from stac.stac_voxel import STACVoxelKV
    from stac.voxel import BinaryVoxel
    return BinaryVoxel, VoxelKVMerger, STACVoxelKV


def _pool_snapshot(m, V):
    """Slot maps and dense contents of a reference VoxelKVMerger over the first V voxels."""
    import torch
    out = {}
    H = m.H
    for tag, wrap in (("buf", m.buffer), ("piv", m.pivots)):
        be = wrap.backend
        Va = be.S_tot // H
        out[tag + "_state"] = be.row_state.view(H, Va)[:, :V].numpy().copy()
        out[tag + "_offset"] = be.row_offset.view(H, Va)[:, :V].numpy().copy()
        out[tag + "_seg"] = be.row_seg.view(H, Va, be.R)[:, :V].numpy().copy()
        out[tag + "_top"] = np.int64(be.seg_top)
        out[tag + "_free"] = np.array(be.seg_free_list, np.int32)
        rows = (torch.arange(H)[:, None] * Va + torch.arange(V)[None, :]).reshape(-1)
        pack = wrap.read_rows_dict(rows)
        for f, t in pack.items():
            if f == "M":
                continue
            out[f"{tag}_{f}"] = t.float().numpy().reshape((H, V) + tuple(t.shape[1:])).copy()
    hv = torch.stack([m.rows_over // m._overflow_alloc, m.rows_over % m._overflow_alloc], 1)
    out["over_hv"] = hv.numpy().astype(np.int64)
    out["over_K"] = m.K_over.float().numpy().copy()
    out["over_V"] = m.V_over.float().numpy().copy()
    out["over_S"] = m.S_over.float().numpy().copy()
    return out


def gen_voxel(BinaryVoxel):
    import torch
    c = cases.VOXEL
    vm = BinaryVoxel(voxel_size=c["voxel_size"], device="cpu")
    out = {}
    for step, pts in enumerate(cases.voxel_points()):
        p = torch.from_numpy(pts)
        ijk = torch.floor(p / torch.tensor(c["voxel_size"], dtype=torch.float32)).to(torch.int32)
        ids = vm.upsert(ijk)
        out[f"ijk_{step}"] = ijk.numpy().copy()
        out[f"ids_{step}"] = ids.numpy().copy()
        q = torch.unique(ids)[: c["n_query"]]
        nb, _, _ = vm.neighbors(voxel_ids=q, radius_m=2 * c["voxel_size"], include_self=True)
        nb = torch.unique(nb[nb >= 0])
        out[f"query_{step}"] = q.numpy().copy()
        out[f"nbr_{step}"] = nb.numpy().astype(np.int64)
    out["keys_1d"] = vm._voxel_keys_1d.numpy().copy()
    out["table_ijk"] = vm._voxel_keys.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "voxel_table.npz"), **out)


def gen_merger(BinaryVoxel, VoxelKVMerger, name):
    import torch
    c = cases.MERGER[name]
    tdt = torch.float32 if c["dtype"] == "f32" else torch.bfloat16
    vm = BinaryVoxel(voxel_size=c["voxel_size"], device="cpu")
    m = VoxelKVMerger(num_heads=c["H"], head_dim=c["D"], init_voxels=c["init_voxels"],
                      pivot_cap=c["P"], budget_cap=c["B"], sim_thresh=c["sim"],
                      replace_thresh=c["replace"], score_thresh=c["score"], dtype=tdt,
                      device=torch.device("cpu"), backend="python", allocator="segment",
                      seg_size=1, slab_growth=1024, slab_cap=10000)
    out = {}
    for step, (pts, K, V, S) in enumerate(cases.merger_inputs(name)):
        ijk = torch.floor(torch.from_numpy(pts) / torch.tensor(c["voxel_size"])).to(torch.int32)
        ids = vm.upsert(ijk)
        H, N = c["H"], pts.shape[0]
        VX = ids.view(1, -1).expand(H, N).contiguous()
        bad = cases.merger_invalid_mask(name, step, N)
        VX = VX.clone()
        VX[:, torch.from_numpy(bad)] = -1
        m.insert_and_merge(torch.from_numpy(K).to(tdt), torch.from_numpy(V).to(tdt),
                           torch.from_numpy(S), torch.arange(N).expand(H, N).contiguous(), VX,
                           num_voxels=vm.get_voxel_num(), mode="default")
        snap = _pool_snapshot(m, vm.get_voxel_num())
        full = step in c["dump_steps"]
        for k, v in snap.items():
            if full or k.endswith(("_state", "_offset", "_seg", "_top", "_free", "over_hv")):
                out[f"s{step}_{k}"] = v
        out[f"s{step}_V"] = np.int64(vm.get_voxel_num())
    for tag, (q, R, rb) in c["retrieve"].items():
        qs = None if q is None else torch.from_numpy(cases.retrieve_query(name, tag))
        Kr, Vr, Mr, Br = m.retrieve(voxel_ids=qs, return_buf=rb, retrieve_size=R)
        out[f"ret_{tag}_K"] = Kr.float().numpy()
        out[f"ret_{tag}_V"] = Vr.float().numpy()
        out[f"ret_{tag}_M"] = Mr.numpy()
        out[f"ret_{tag}_B"] = Br.numpy()
    np.savez_compressed(os.path.join(HERE, f"merger_{name}.npz"), **out)


def gen_manager(STACVoxelKV):
    import torch
    c = cases.MANAGER
    kv = STACVoxelKV(num_layers=c["L"], num_heads=c["H"], head_dim=c["D"],
                     token_per_frame=c["tpf"], buffer_size=c["buffer"], chunk_size=c["chunk"],
                     recent_size=c["window"], pinned_idx=[0], hh_size=c["hh"], temperature=0.9,
                     device=torch.device("cpu"), dtype=torch.float32, voxel_size=c["voxel_size"],
                     init_voxels=c["init_voxels"], voxel_buf_cap=8, voxel_piv_cap=4,
                     voxel_backend="python", sim_threshold=0.8, replace_threshold=0.8,
                     score_threshold=0.2, slab_growth=1024, slab_cap=10000, seg_size=1,
                     retrieval_size=c["retrieval"], allocator="segment", attn_backend="cuda")
    kv.reset()
    out = {}
    for step, (k, v, cs, pts, mask) in enumerate(cases.manager_inputs()):
        Tq = k.shape[2]
        for l in range(c["L"]):
            kv.append_kv(torch.from_numpy(k[l])[None], torch.from_numpy(v[l])[None], l)
            kv._last_query_offset[l] = Tq
            T_live = kv._offset_hot[l]
            kv._update_scores(torch.from_numpy(cs[l][:, :T_live])[None, :, None, :], l)
        kv.append_positions(torch.from_numpy(pts), torch.from_numpy(mask))
        if step in c["retrieve_steps"]:
            kv.retrieve_kv(0, return_buf=True)
            out[f"s{step}_ret_T"] = np.array(kv._offset_retrieval, np.int64)
            if kv._offset_retrieval[0] > 0:
                out[f"s{step}_ret_K"] = torch.stack(kv.key_cache_retrieval).numpy()
                out[f"s{step}_ret_bias"] = torch.stack(kv._bias_retrieval).numpy()
        rid = kv._recent_voxel_ids
        out[f"s{step}_recent"] = (np.empty(0, np.int64) if rid is None
                                  else np.unique(rid.numpy().astype(np.int64)))
        kv.prune_kv()
        T = kv._offset_hot[0]
        out[f"s{step}_T"] = np.int64(T)
        out[f"s{step}_TI"] = kv._token_indices_hot[:, :, :T].numpy().copy()
        out[f"s{step}_VX"] = kv._token_voxel_indices[:, :, :T].numpy().copy()
        out[f"s{step}_S"] = kv._scores_hot[:, :, :T].numpy().copy()
        snap = _pool_snapshot(kv._vstore, kv._vstore._voxel_offset)
        out[f"s{step}_Vused"] = np.int64(kv._vstore._voxel_offset)
        for key, val in snap.items():
            if key.endswith(("_state", "_offset", "_seg", "_top", "_free", "over_hv")):
                out[f"s{step}_{key}"] = val
    out["final_K"] = kv.key_cache_hot[:, :, :T].numpy().copy()
    np.savez_compressed(os.path.join(HERE, "manager_trace.npz"), **out)


def gen_attention():
    """fp32 attention with column sums computed with torch ops, following the reference's
    own check (stac/flash_attn_triton.py:1018-1036)."""
    import torch
    out = {}
    for name in cases.ATTENTION:
        q, k, v, bias = cases.attention_inputs(name)
        qt = torch.from_numpy(q).transpose(0, 1)
        kt = torch.from_numpy(k).transpose(0, 1)
        vt = torch.from_numpy(v).transpose(0, 1)
        s = torch.matmul(qt, kt.transpose(-2, -1)) * (q.shape[-1] ** -0.5)
        if bias is not None:
            s = s + torch.from_numpy(bias).unsqueeze(1)
        lse = torch.logsumexp(s, dim=-1)
        p = torch.softmax(s, dim=-1)
        out[f"{name}_colsum"] = p.sum(dim=1).numpy()
        out[f"{name}_lse"] = lse.numpy()
        out[f"{name}_out"] = torch.matmul(p, vt).transpose(0, 1).numpy()
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **out)


def gen_pointmap(ref_path):
    """StreamSession.get_pointmap (stream_session.py:213-256) called unbound with a stand-in for
    `self` that carries only the patch size; CPU."""
    import types
    import torch
    sys.path.insert(0, ref_path)
    from stream_session import StreamSession
    out = {}
    for name, c in cases.POINTMAP.items():
        wp, cf = cases.pointmap_inputs(name)
        me = types.SimpleNamespace(model=types.SimpleNamespace(point_head=types.SimpleNamespace(patch_size=c["patch"])))
        outputs = {"world_points": torch.from_numpy(wp)[None], "world_points_conf": torch.from_numpy(cf)[None]}
        pts, mask = StreamSession.get_pointmap(me, outputs, conf_threshold=c["conf_threshold"],
                                               special_tokens_size=c["special"])
        out[f"{name}_pts"] = pts.numpy()
        out[f"{name}_mask"] = mask.numpy()
    np.savez_compressed(os.path.join(HERE, "pointmap.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python make_golden.py <path to a checkout of Rainzor/STAC>")
    ref = sys.argv[1]
    BinaryVoxel, VoxelKVMerger, STACVoxelKV = _import_reference(ref)
    gen_voxel(BinaryVoxel)
    for nm in cases.MERGER:
        gen_merger(BinaryVoxel, VoxelKVMerger, nm)
    gen_manager(STACVoxelKV)
    gen_attention()
    gen_pointmap(ref)
    print("golden fixtures written to", HERE)
