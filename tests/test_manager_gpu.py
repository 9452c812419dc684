"""The drop-in manager classes on the GPU against the oracle manager, chunk by chunk, in the
reference's call order.  Column sums are injected through `_update_scores` (as the reference's
own CPU trace does) so that both sides select from identical scores; a second test drives the
real attention kernel and checks the scores it produces."""

import numpy as np
import pytest
import torch

import cases
from oracle.attention import attn_colsum as oracle_attn
from oracle.manager import StacManager

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make(c, **over):
    from stac_b200.stac import STACVoxelKV
    kw = dict(num_layers=c["L"], num_heads=c["H"], head_dim=c["D"], token_per_frame=c["tpf"],
              buffer_size=c["buffer"], chunk_size=c["chunk"], recent_size=c["window"], pinned_idx=[0],
              hh_size=c["hh"], temperature=0.9, device=torch.device(DEV), dtype=torch.bfloat16,
              voxel_size=c["voxel_size"], init_voxels=c["init_voxels"], voxel_buf_cap=8, voxel_piv_cap=4,
              voxel_backend="cuda", sim_threshold=0.8, replace_threshold=0.8, score_threshold=0.2,
              slab_growth=1024, slab_cap=10000, seg_size=1, retrieval_size=c["retrieval"],
              allocator="segment", attn_backend="cuda", some_unknown_cli_flag=1)
    kw.update(over)
    kv = STACVoxelKV(**kw)
    kv.reset()
    return kv


def test_trace_matches_oracle():
    c = cases.MANAGER_GPU
    kv = _make(c)
    ref = StacManager(c["L"], c["H"], c["D"], c["tpf"], c["buffer"], chunk_size=c["chunk"],
                      recent_size=c["window"], pinned_idx=(0,), hh_size=c["hh"], temperature=0.9,
                      voxel_size=c["voxel_size"], init_voxels=c["init_voxels"],
                      retrieval_size=c["retrieval"], dtype="bf16")
    L, H, D = c["L"], c["H"], c["D"]
    retrieved = 0
    for step, (k, v, cs, pts, mask) in enumerate(cases.manager_inputs(c)):
        Tq = k.shape[2]
        for l in range(L):
            tk = torch.from_numpy(k[l]).to(torch.bfloat16)
            tv = torch.from_numpy(v[l]).to(torch.bfloat16)
            kv.append_kv(tk[None].to(DEV), tv[None].to(DEV), l)
            ref.append_kv(tk.float().numpy(), tv.float().numpy(), l)
            T_live = kv._offset_hot[l]
            kv._last_query_offset[l] = Tq
            kv._update_scores(torch.from_numpy(cs[l][:, :T_live])[None, :, None, :].to(DEV), l)
            ref.update_scores(cs[l][:, :T_live], l, Tq)
        kv.append_positions(torch.from_numpy(pts).to(DEV), torch.from_numpy(mask).to(DEV))
        ref.append_positions(pts, mask)
        if ref.recent_ids is not None:
            ids, cnt = kv._recent_voxel_ids
            n = int(cnt.item())
            assert np.array_equal(ids[:n].cpu().numpy().astype(np.int64), np.unique(ref.recent_ids)), step
        if step in c["retrieve_steps"]:
            for l in range(L):
                kv.retrieve_kv(l, return_buf=True)
            ref.ret = None
            ref.retrieve(return_buf=True)
            R = kv.retrieval_token_size
            assert kv.get_retrieval_size() == [R] * L
            Kr, Vr, Br, Mr, _ = ref.ret
            gk = torch.stack(kv.key_cache_retrieval).float().cpu().numpy().reshape(L * H, R, D)
            gb = torch.stack(kv._bias_retrieval).cpu().numpy().reshape(L * H, R)
            fin = np.isfinite(Br)
            assert np.array_equal(np.isfinite(gb), fin), step
            np.testing.assert_allclose(gb[fin], Br[fin], rtol=1e-5, atol=1e-6)
            np.testing.assert_allclose(gk, Kr, rtol=8e-3, atol=1e-3)
            retrieved += int(fin.sum())
        kv.prune_kv()
        ref.prune()
        T = ref.off[0]
        assert kv.get_offset() == [T] * L, step
        assert np.array_equal(kv._token_indices_hot[:, :, :T].cpu().numpy(), ref.TI[:, :, :T]), step
        assert np.array_equal(kv._token_voxel_indices[:, :, :T].cpu().numpy(), ref.VX[:, :, :T]), step
        assert np.array_equal(kv._scores_hot[:, :, :T].cpu().numpy(), ref.S[:, :, :T]), step
        assert np.array_equal(kv.key_cache_hot[:, :, :T].float().cpu().numpy(), ref.K[:, :, :T]), step
        assert bool((kv._token_indices_hot[:, :, T:] == -1).all())
        snap = kv._vstore.snapshot()
        sm = ref.merger.slot_map()
        for key in ("buf_offset", "buf_seg", "piv_offset", "piv_seg"):
            assert np.array_equal(snap[key], sm[key]), (step, key)
        assert np.array_equal(snap["buf_free"], sm["buf_free"]), step
    kv.check_status()
    assert retrieved > 0
    det = kv.get_memory_details()
    assert det["voxel_pivot_usage"] > 0 and det["total_usage"] > 0
    assert kv.get_merger_info()["used_voxels"] == ref.merger.V_used
    kv.free()


def test_attention_drives_scores():
    """decode_sparse_attn over [hot | retrieved] updates the hot scores with the column sums."""
    c = dict(cases.MANAGER_GPU)
    kv = _make(c)
    L, H, D, tpf = c["L"], c["H"], c["D"], c["tpf"]
    rs = np.random.RandomState(4)
    Tn = c["chunk"] * tpf
    k = torch.from_numpy(rs.randn(H, Tn, D).astype(np.float32)).to(torch.bfloat16)
    v = torch.from_numpy(rs.randn(H, Tn, D).astype(np.float32)).to(torch.bfloat16)
    q = torch.from_numpy(rs.randn(Tn, H, D).astype(np.float32)).to(torch.bfloat16)
    kv.append_kv(k[None].to(DEV), v[None].to(DEV), 0)
    # fake retrieved pivots for layer 0
    R = 50
    kr = torch.from_numpy(rs.randn(H, R, D).astype(np.float32)).to(torch.bfloat16)
    vr = torch.from_numpy(rs.randn(H, R, D).astype(np.float32)).to(torch.bfloat16)
    br = np.log(rs.randint(1, 9, size=(H, R)).astype(np.float32))
    br[:, -7:] = -np.inf
    kv.key_cache_retrieval[0], kv.value_cache_retrieval[0] = kr.to(DEV), vr.to(DEV)
    kv._bias_retrieval[0] = torch.from_numpy(br).to(DEV)
    kv._offset_retrieval[0] = R
    out = kv.decode_sparse_attn(q[None].to(DEV), 0)
    kv.check_status()
    k_all = torch.cat([k, kr], 1).float().numpy().transpose(1, 0, 2)
    v_all = torch.cat([v, vr], 1).float().numpy().transpose(1, 0, 2)
    b_all = np.concatenate([np.zeros((H, Tn), np.float32), br], 1)
    o_ref, _, cs_ref = oracle_attn(q.float().numpy(), k_all, v_all, b_all)
    assert out.shape == (1, Tn, H, D)
    assert np.abs(out[0].float().cpu().numpy() - o_ref).max() <= 2e-2
    s_ref = cs_ref[:, :Tn] * np.float32(Tn) / np.float32(Tn)
    np.testing.assert_allclose(kv.get_scores()[0, :, :Tn].cpu().numpy(), s_ref, rtol=1e-3, atol=1e-6)
    assert float(kv._scores_hot_count[0, :, :Tn].min()) == 1.0
    kv.free()


def test_float16_is_converted_at_the_manager_boundary():
    """dtype=float16 (the bare default of the reference's register_kv_mgr) is accepted: the cache
    and the kernels are bf16, keys / values / queries are converted on the way in and the output
    comes back as float16, equal to the bf16 manager's output on the same (bf16-representable) inputs."""
    from stac_b200.stac import HeavyHittersKV
    L, H, D, tpf = 1, 2, 64, 16
    common = dict(num_layers=L, num_heads=H, head_dim=D, token_per_frame=tpf, chunk_size=1, recent_size=2,
                  pinned_idx=[0], device=torch.device(DEV), buffer_size=5, hh_size=1, temperature=0.9)
    with pytest.warns(UserWarning, match="float16"):
        a = HeavyHittersKV(dtype=torch.float16, **common)
    b = HeavyHittersKV(dtype=torch.bfloat16, **common)
    a.reset()
    b.reset()
    g = torch.Generator().manual_seed(4)
    for _ in range(3):
        k = (torch.randn(1, H, tpf, D, generator=g) / 2).to(torch.bfloat16)
        v = torch.randn(1, H, tpf, D, generator=g).to(torch.bfloat16)
        q = (torch.randn(1, tpf, H, D, generator=g) / 2).to(torch.bfloat16)
        a.append_kv(k.to(torch.float16).to(DEV), v.to(torch.float16).to(DEV), 0)
        b.append_kv(k.to(DEV), v.to(DEV), 0)
        oa = a.decode_sparse_attn(q.to(torch.float16).to(DEV), 0)
        ob = b.decode_sparse_attn(q.to(DEV), 0)
        assert oa.dtype == torch.float16 and ob.dtype == torch.bfloat16
        assert torch.allclose(oa.float(), ob.float(), rtol=0, atol=1e-6)   # bf16 -> fp16 is exact above 2^-14
    assert torch.equal(a.get_scores()[0], b.get_scores()[0])
    with pytest.raises(ValueError):
        HeavyHittersKV(dtype=torch.float32, **common)


def test_window_manager_and_h2o_manager():
    """KVManager (recent + pinned) and HeavyHittersKV (no voxel memory) prune like the oracle."""
    from oracle.manager import h2o_keep_indices
    from stac_b200.stac import HeavyHittersKV, KVManager
    L, H, D, tpf = 2, 2, 64, 16
    rs = np.random.RandomState(2)
    common = dict(num_layers=L, num_heads=H, head_dim=D, token_per_frame=tpf, chunk_size=1, recent_size=2,
                  pinned_idx=[0], device=torch.device(DEV), dtype=torch.bfloat16)
    win = KVManager(buffer_size=4, **common)
    hh = HeavyHittersKV(buffer_size=5, hh_size=1, temperature=0.9, **common)
    win.reset()
    hh.reset()
    scores_ref = np.zeros((L, H, 5 * tpf), np.float32)
    ti_ref = np.full((L, H, 5 * tpf), -1, np.int64)
    T_ref, last = 0, 0
    for frame in range(7):
        for l in range(L):
            k = torch.from_numpy(rs.randn(1, H, tpf, D).astype(np.float32)).to(torch.bfloat16).to(DEV)
            win.append_kv(k, k, l)
            hh.append_kv(k, k, l)
        ti_ref[:, :, T_ref:T_ref + tpf] = np.arange(frame * tpf, (frame + 1) * tpf)
        T_ref += tpf
        q = torch.from_numpy(rs.randn(1, tpf, H, D).astype(np.float32)).to(torch.bfloat16).to(DEV)
        assert win.decode_sparse_attn(q, 0).shape == (1, tpf, H, D)
        for l in range(L):
            cs = rs.rand(H, T_ref).astype(np.float32)
            hh._last_query_offset[l] = tpf
            hh._update_scores(torch.from_numpy(cs)[None, :, None, :].to(DEV), l)
            s = cs * np.float32(T_ref) / np.float32(tpf)
            scores_ref[l, :, last:T_ref] = s[:, last:]
            scores_ref[l, :, :last] = scores_ref[l, :, :last] * np.float32(0.9) + s[:, :last]
        last = T_ref
        win.prune_kv()
        hh.prune_kv()
        keep = h2o_keep_indices(scores_ref, T_ref, 2 * tpf, np.arange(tpf), tpf, 4 * tpf)
        if keep is not None:
            Tp = keep.shape[-1]
            ti_ref[:, :, :Tp] = np.take_along_axis(ti_ref[:, :, :T_ref], keep, 2)
            ti_ref[:, :, Tp:] = -1
            scores_ref[:, :, :Tp] = np.take_along_axis(scores_ref[:, :, :T_ref], keep, 2)
            scores_ref[:, :, Tp:] = 0
            T_ref = Tp
            last = min(last, Tp)
        assert hh.get_offset() == [T_ref] * L
        assert np.array_equal(hh.get_token_indices().numpy(), ti_ref)
        assert np.array_equal(hh.get_scores().cpu().numpy(), scores_ref)
        assert win.get_offset()[0] <= 3 * tpf + tpf
    assert win.get_offset() == [3 * tpf] * L
    first = win.get_token_indices()[0, 0, : 3 * tpf].numpy()
    assert np.array_equal(first[:tpf], np.arange(tpf)) and np.array_equal(first[tpf:], np.arange(5 * tpf, 7 * tpf))


def test_cpu_spill_of_the_window_manager():
    """Buffers longer than gpu_limit frames: the oldest tokens of an append that does not fit go to
    the host buffer, plain attention still sees them, the host buffer raises when full
    (stac/kv_manager.py:227-360)."""
    import warnings
    from stac_b200.stac import KVManager
    dev = torch.device("cuda:0")
    tpf, H, D, L = 40, 2, 64, 2
    mgr = KVManager(num_layers=L, num_heads=H, head_dim=D, token_per_frame=tpf, chunk_size=1, buffer_size=5,
                    recent_size=1, pinned_idx=[0], dtype=torch.bfloat16, device=dev, gpu_limit=2)
    mgr.reset()
    assert mgr.reserved_buffer_token_size == 2 * tpf and mgr.reserved_buffer_token_size_cpu == 3 * tpf
    g = torch.Generator().manual_seed(4)
    ks, vs = [], []

    def append(frames):
        k = torch.randn(L, 1, H, frames * tpf, D, generator=g).to(torch.bfloat16)
        v = torch.randn(L, 1, H, frames * tpf, D, generator=g).to(torch.bfloat16)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            for l in range(L):
                mgr.append_kv(k[l].to(dev), v[l].to(dev), l)
        ks.append(k), vs.append(v)

    append(1)                       # fits
    assert mgr.get_offset() == [tpf] * L and mgr.get_offset_cpu() == [0] * L and not mgr.use_cpu
    append(3)                       # one frame of room: the first two frames spill, the last stays
    assert mgr.get_offset() == [2 * tpf] * L and mgr.get_offset_cpu() == [2 * tpf] * L and mgr.use_cpu
    ti = mgr.get_token_indices()
    assert np.array_equal(ti[0, 0].numpy(), np.r_[np.arange(tpf), np.arange(3 * tpf, 4 * tpf)])
    used, alloc = mgr.get_cpu_memory_usage()
    assert used == pytest.approx(L * 2 * H * 2 * tpf * D * 2 / 1024.0 ** 2) and alloc > used
    q = torch.randn(1, 50, H, D, generator=g).to(torch.bfloat16)
    for l in range(L):
        out = mgr.decode_sparse_attn(q.to(dev), l)
        torch.cuda.synchronize()
        k_all = torch.cat([x[l, 0] for x in ks], dim=1).float().numpy().transpose(1, 0, 2)   # [T, H, D]
        v_all = torch.cat([x[l, 0] for x in vs], dim=1).float().numpy().transpose(1, 0, 2)
        o_ref, _, _ = oracle_attn(q[0].float().numpy(), k_all, v_all, None)
        assert np.abs(out[0].float().cpu().numpy() - o_ref).max() <= 2e-2
    mgr.check_status() if hasattr(mgr, "check_status") else None
    append(1)                       # GPU part full: everything goes to the host (3 of 3 frames now)
    assert mgr.get_offset_cpu() == [3 * tpf] * L
    with pytest.raises(RuntimeError, match="CPU buffer overflow"):
        append(1)


def _drive(kv, c, steps, start=0, log=None):
    """Steps [start, steps) of the seeded manager trace (column sums injected, retrieval on the
    configured steps); appends the retrieved pivots of every retrieval to `log`."""
    L = c["L"]
    for step, (k, v, cs, pts, mask) in enumerate(cases.manager_inputs(c)):
        if step < start:
            continue
        if step >= steps:
            break
        Tq = k.shape[2]
        for l in range(L):
            tk = torch.from_numpy(k[l]).to(torch.bfloat16)
            tv = torch.from_numpy(v[l]).to(torch.bfloat16)
            kv.append_kv(tk[None].to(DEV), tv[None].to(DEV), l)
            T_live = kv._offset_hot[l]
            kv._last_query_offset[l] = Tq
            kv._update_scores(torch.from_numpy(cs[l][:, :T_live])[None, :, None, :].to(DEV), l)
        kv.append_positions(torch.from_numpy(pts).to(DEV), torch.from_numpy(mask).to(DEV))
        if step in c["retrieve_steps"]:
            for l in range(L):
                kv.retrieve_kv(l, return_buf=True)
            if log is not None:
                log.append((torch.stack(kv.key_cache_retrieval).float().cpu().numpy(),
                            torch.stack(kv._bias_retrieval).cpu().numpy()))
        kv.prune_kv()


def _full_state(kv):
    T = kv.get_offset()[0]
    snap = kv._vstore.snapshot()
    out = {"ti": kv._token_indices_hot[:, :, :T].cpu().numpy(), "vx": kv._token_voxel_indices[:, :, :T].cpu().numpy(),
           "sc": kv._scores_hot[:, :, :T].cpu().numpy(), "cn": kv._scores_hot_count[:, :, :T].cpu().numpy(),
           "k": kv.key_cache_hot[:, :, :T].float().cpu().numpy(), "v": kv.value_cache_hot[:, :, :T].float().cpu().numpy(),
           "n_vox": np.array(kv._vm.get_voxel_num()), "keys": kv._vm.get_voxel_keys_1d().cpu().numpy()}
    for key, val in snap.items():
        out["mem_" + key] = np.asarray(val)
    return out


def test_checkpoint_resume_continues_with_the_same_bits(tmp_path):
    """A stream saved after step 9 (between a retrieval and the next attention) and restored into a
    new manager ends with exactly the state of the uninterrupted stream."""
    from stac_b200.stac.checkpoint import load_state, save_state
    c = cases.MANAGER_GPU
    cut = 9
    a_log, b_log = [], []
    a = _make(c)
    _drive(a, c, c["steps"], log=a_log)
    want = _full_state(a)
    b = _make(c)
    _drive(b, c, cut, log=b_log)
    path = str(tmp_path / "stream_state.pt")
    save_state(b, path)
    b.free()
    r = _make(c)
    load_state(r, path)
    assert r._processed_frames == cut * c["chunk"]
    _drive(r, c, c["steps"], start=cut, log=b_log)
    r.check_status()
    got = _full_state(r)
    assert set(got) == set(want)
    for key in want:
        assert np.array_equal(got[key], want[key]), key
    assert len(a_log) == len(b_log) and len(a_log) > 2
    for (ka, ba), (kb, bb) in zip(a_log, b_log):
        assert np.array_equal(ka, kb) and np.array_equal(ba, bb)
    with pytest.raises(ValueError):
        _make(c, buffer_size=c["buffer"] + 1).load_state_dict(torch.load(path, weights_only=True))


def test_long_stream_with_bounded_voxel_memory():
    """400 frames through a narrow manager (2 layers x 4 heads) with real attention every step and
    voxel-memory pools far smaller than the stream needs: no device error, the pools stay inside
    their bounds, rows are trimmed and retrieval returns pivots."""
    from stac_b200.stac import STACVoxelKV
    import bench
    dev = torch.device(DEV)
    L, H, D, tpf, chunk = 2, 4, 64, 1041, 4
    max_buf, max_piv = 1_000_000, 100_000
    kv = STACVoxelKV(num_layers=L, num_heads=H, head_dim=D, token_per_frame=tpf, buffer_size=chunk + 1 + 4 + 1,
                     chunk_size=chunk, recent_size=4, pinned_idx=[0], hh_size=1, temperature=0.9, device=dev,
                     dtype=torch.bfloat16, voxel_size=0.05, init_voxels=4096, voxel_buf_cap=8, voxel_piv_cap=4,
                     retrieval_size=1, max_buffer_slots=max_buf, max_pivot_slots=max_piv)
    kv.reset()
    n_chunks = 100
    pts = bench.synth_points(n_chunks, seed=3)
    g = torch.Generator(device="cpu").manual_seed(5)
    Tq = chunk * tpf
    q = (torch.randn(L, 1, Tq, H, D, generator=g) / 2).to(torch.bfloat16).to(dev)
    k = (torch.randn(L, 1, H, Tq, D, generator=g) / 2).to(torch.bfloat16).to(dev)
    v = (torch.randn(L, 1, H, Tq, D, generator=g) / 8).to(torch.bfloat16).to(dev)
    valid_retrieved = 0
    for i in range(n_chunks):
        for l in range(L):
            kv.append_kv(k[l].roll(i, dims=2), v[l].roll(i, dims=2), l)
            out = kv.decode_sparse_attn(q[l], l)
        kv.append_positions(torch.from_numpy(pts[i][0]).to(dev), torch.from_numpy(pts[i][1]).to(dev))
        if bench.retrieval_due(i):
            for l in range(L):
                kv.retrieve_kv(l, return_buf=True)
            valid_retrieved = max(valid_retrieved, int(torch.isfinite(torch.stack(kv._bias_retrieval)).sum()))
        kv.prune_kv()
    kv.check_status()
    info = kv.get_merger_info()
    assert info["buffer_pool_used"] <= max_buf and info["pivot_pool_used"] <= max_piv
    assert info["dropped_tokens"] > 0 and info["pivot_pool_used"] > 0
    assert info["used_voxels"] > 10_000
    assert bool(torch.isfinite(out.float()).all())
    R = kv.retrieval_token_size
    assert kv.get_retrieval_size() == [R] * L
    # (once the pools are full, rows of new voxels are the first to be trimmed, so late retrievals
    # around the newest frames may find no pivot at all; earlier ones must have)
    assert bool(torch.isfinite(torch.stack(kv.key_cache_retrieval).float()).all()) and valid_retrieved > 0
    # the pools themselves never grow past their bounds (the row maps grow with the voxel count)
    assert kv._vstore._buf_cap <= max_buf and kv._vstore._piv_cap <= max_piv
    kv.free()


def test_steady_state_steps_never_wait_for_the_gpu():
    """The reference's loop blocks on the GPU several times per chunk (.item(), .cpu().tolist(),
    a stream synchronise inside the merger, stream_session.py:451-553).  Here a steady-state
    chunk (append_kv + attention per layer, append_positions, retrieve, prune with eviction
    merge) must not contain a single implicit synchronisation: torch raises on any under
    set_sync_debug_mode("error").  Counters are read one step late from pinned memory."""
    c = dict(cases.MANAGER_GPU)
    kv = _make(c)
    L, H, D = c["L"], c["H"], c["D"]
    dev = torch.device(DEV)
    inputs = []
    for k, v, cs, pts, mask in cases.manager_inputs(c):
        inputs.append((torch.from_numpy(k).to(torch.bfloat16).to(dev), torch.from_numpy(v).to(torch.bfloat16).to(dev),
                       torch.from_numpy(pts).to(dev), torch.from_numpy(mask).to(dev)))
    g = torch.Generator(device="cpu").manual_seed(5)
    Tq = inputs[0][0].shape[2]
    q = torch.randn(1, Tq, H, D, generator=g).to(torch.bfloat16).to(dev)

    def step(i):
        k, v, pts, mask = inputs[i]
        for l in range(L):
            kv.append_kv(k[l][None], v[l][None], l)
            kv.decode_sparse_attn(q, l)
        kv.append_positions(pts, mask)
        if i >= 6:
            for l in range(L):
                kv.retrieve_kv(l, return_buf=True)
        kv.prune_kv()

    warm = 12                     # past the first evictions, pool growth and scratch sizing
    for i in range(warm):
        step(i)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        for i in range(warm, len(inputs)):
            step(i)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    kv.check_status()
    info = kv.get_merger_info()
    assert info["pivot_pool_used"] > 0 and info["used_voxels"] == kv._vm.get_voxel_num()
    kv.free()
