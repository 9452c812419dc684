"""Parity of the memory-bound kernels (voxel table, H2O selection/compaction, eviction merge,
retrieval) against the CPU oracle, through the C ABI.  Integer outputs bit-exact; merged
values within 1e-3 relative for fp32 pools (bf16 pools: one bf16 ulp)."""

import numpy as np
import pytest
import torch

import cases
from oracle.manager import h2o_keep_indices
from oracle.pool import VoxelMerger
from oracle.voxel import VoxelTable, quantize

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _table(cap=1 << 12):
    from stac_b200 import ops
    from stac_b200.stac.voxel import BinaryVoxel
    st = ops.DeviceStatus(torch.device(DEV))
    return BinaryVoxel(0.05, DEV, capacity=cap, status=st), st


def test_voxel_upsert_and_neighbors_match_oracle():
    t_gpu, st = _table(cap=256)   # small capacity: exercises growth + rehash
    t_ref = VoxelTable(0.05)
    for step, pts in enumerate(cases.voxel_points()):
        mask = np.ones(pts.shape[0], bool)
        mask[::7] = False
        ids = t_gpu.upsert_points(torch.from_numpy(pts), torch.from_numpy(mask)).cpu().numpy()
        ref = np.full(pts.shape[0], -1, np.int32)
        ref[mask] = t_ref.upsert(quantize(pts, 0.05)[mask])
        assert np.array_equal(ids, ref), step
        assert t_gpu.get_voxel_num() == t_ref.num_voxels
        assert np.array_equal(t_gpu.get_voxel_keys_1d().cpu().numpy(), t_ref.keys)
        assert np.array_equal(t_gpu.get_voxel_keys().cpu().numpy(), t_ref.ijk)
        q = np.unique(ref[ref >= 0])[:80].astype(np.int32)
        nb_ids, nb_cnt = t_gpu.neighbor_ids(torch.from_numpy(q).to(DEV), 2)
        n = int(nb_cnt.item())
        assert np.array_equal(nb_ids[:n].cpu().numpy().astype(np.int64), t_ref.neighbors(q, 2)), step
    st.raise_if_set("voxel")
    all_ids, cnt = t_gpu.neighbor_ids(None, 0, all_ids=True)
    assert int(cnt.item()) == t_ref.num_voxels
    assert np.array_equal(all_ids[: t_ref.num_voxels].cpu().numpy(), np.arange(t_ref.num_voxels))


def test_voxel_cell_boundaries_use_true_division():
    """Points on or next to cell faces: floor(p / 0.05) in fp32, not p * 20."""
    t_gpu, _ = _table()
    k = np.arange(-200, 200, dtype=np.float32)
    pts = np.stack([k * np.float32(0.05), k * np.float32(0.05) + np.float32(1e-7),
                    np.nextafter(k * np.float32(0.05), np.float32(-1e9))], 1).astype(np.float32)
    ids = t_gpu.upsert_points(torch.from_numpy(pts)).cpu().numpy()
    t_ref = VoxelTable(0.05)
    assert np.array_equal(ids, t_ref.upsert(quantize(pts, 0.05)))


def test_upsert_integer_coordinates_entry():
    t_gpu, _ = _table()
    rs = np.random.RandomState(3)
    ijk = rs.randint(-50, 50, size=(3000, 3)).astype(np.int32)
    ids = t_gpu.upsert(torch.from_numpy(ijk)).cpu().numpy()
    assert np.array_equal(ids, VoxelTable(0.05).upsert(ijk))


def test_empty_and_fully_masked_inputs_are_no_ops():
    """Zero points, zero tokens, all-masked points, tokens without a valid voxel, an empty query:
    every entry point returns cleanly and leaves the state untouched."""
    from stac_b200.stac.merger import VoxelKVMerger
    t_gpu, st = _table()
    assert t_gpu.upsert_points(torch.zeros((0, 3))).numel() == 0
    assert t_gpu.upsert(torch.zeros((0, 3), dtype=torch.int32)).numel() == 0
    ids = t_gpu.upsert_points(torch.rand(50, 3), torch.zeros(50, dtype=torch.bool))
    assert (ids.cpu().numpy() == -1).all() and t_gpu.get_voxel_num() == 0
    _, cnt = t_gpu.neighbor_ids(torch.zeros(0, dtype=torch.int32, device=DEV), 2)
    assert int(cnt.item()) == 0
    g = VoxelKVMerger(2, 64, init_voxels=8, pivot_cap=4, budget_cap=8, sim_thresh=0.8, replace_thresh=0.8,
                      score_thresh=0.2, dtype=torch.bfloat16, device=DEV, status=st)
    z = torch.zeros((2, 0, 64), dtype=torch.bfloat16, device=DEV)
    assert g.insert_and_merge(z, z, torch.zeros((2, 0), device=DEV), None,
                              torch.zeros((2, 0), dtype=torch.int32, device=DEV), 0) == {}
    k = torch.randn((2, 10, 64), device=DEV).to(torch.bfloat16)
    g.insert_and_merge(k, k, torch.rand((2, 10), device=DEV), None,
                       torch.full((2, 10), -1, dtype=torch.int32, device=DEV), 4)
    info = g.info()
    assert info["buffer_pool_used"] == 0 and info["pivot_pool_used"] == 0
    K, V, M, B = g.retrieve(torch.zeros(0, dtype=torch.int64), True, 16)
    assert K.shape == (2, 16, 64) and not bool(M.any()) and bool(torch.isinf(B).all())
    st.raise_if_set("empty inputs")


def test_upsert_of_a_long_chunk_sorts_its_new_keys_outside_shared_memory():
    """More new voxels in one call than the in-CTA sort holds (16 384): 40 frames of 1041 points
    on unseen ground, then a second call that mixes known and new voxels."""
    t_gpu, st = _table(cap=1 << 10)
    t_ref = VoxelTable(0.05)
    rs = np.random.RandomState(11)
    for step, (n, spread) in enumerate([(40 * 1041, 6.0), (125 * 1041, 7.0), (20000, 7.0)]):
        pts = rs.uniform(-spread, spread, size=(n, 3)).astype(np.float32)
        mask = rs.rand(n) > 0.05
        ids = t_gpu.upsert_points(torch.from_numpy(pts), torch.from_numpy(mask)).cpu().numpy()
        ref = np.full(n, -1, np.int32)
        n_before = t_ref.num_voxels
        ref[mask] = t_ref.upsert(quantize(pts, 0.05)[mask])
        assert t_ref.num_voxels - n_before > 16384, "the case must exceed the shared-memory sort"
        assert np.array_equal(ids, ref), step
        assert t_gpu.get_voxel_num() == t_ref.num_voxels
    st.raise_if_set("voxel")
    assert np.array_equal(t_gpu.get_voxel_keys_1d().cpu().numpy(), t_ref.keys)
    with pytest.raises(ValueError):
        t_gpu.upsert_points(torch.zeros((131073, 3)))


@pytest.mark.parametrize("T,n_recent,n_pinned,k", [(700, 200, 100, 150), (15615, 8328, 1041, 2082),
                                                     (333, 50, 0, 1), (1200, 100, 37, 1063)])
def test_h2o_select_bit_exact(T, n_recent, n_pinned, k):
    from stac_b200 import _lib
    from stac_b200._lib import ptr, stream_ptr
    rs = np.random.RandomState(T)
    rows, stride = 12, T + 5
    scores = rs.rand(rows, stride).astype(np.float32)
    scores[3, : T // 2] = 0.25          # heavy ties: lower position wins
    scores[4, :T] = 0.0
    pinned = np.arange(n_pinned)
    keep_ref = h2o_keep_indices(scores, T, n_recent, pinned, k, 0)
    base = np.zeros(T, np.uint8)
    base[T - n_recent:] = 1
    base[pinned] = 1
    n_keep = int(base.sum()) + k
    assert keep_ref.shape == (rows, n_keep)
    d_scores = torch.from_numpy(scores).to(DEV)
    keep = torch.empty((rows, n_keep), dtype=torch.int32, device=DEV)
    drop = torch.empty((rows, T - n_keep), dtype=torch.int32, device=DEV)
    rc = _lib.lib().stac_h2o_select(ptr(d_scores), stride, rows, ptr(torch.from_numpy(base).to(DEV)), T, n_keep,
                                    ptr(keep), ptr(drop), stream_ptr())
    assert rc == 0
    keep, drop = keep.cpu().numpy(), drop.cpu().numpy()
    assert np.array_equal(keep, keep_ref)
    for r in range(rows):
        full = np.sort(np.concatenate([keep[r], drop[r]]))
        assert np.array_equal(full, np.arange(T))
        assert np.all(np.diff(drop[r]) > 0)


def test_scores_update_and_compact():
    from stac_b200 import _lib
    from stac_b200._lib import ptr, stream_ptr
    rs = np.random.RandomState(8)
    H, Tb, T_live, old_T, Tq, D = 3, 500, 420, 300, 84, 64
    colsum = rs.rand(H, T_live).astype(np.float32)
    scores = rs.rand(H, Tb).astype(np.float32)
    counts = rs.randint(0, 5, size=(H, Tb)).astype(np.float32)
    ref_s, ref_c = scores.copy(), counts.copy()
    s = colsum * np.float32(T_live) / np.float32(Tq)
    ref_s[:, old_T:T_live] = s[:, old_T:]
    ref_s[:, :old_T] = ref_s[:, :old_T] * np.float32(0.9) + s[:, :old_T]
    ref_c[:, :T_live] += 1
    d_s, d_c = torch.from_numpy(scores).to(DEV), torch.from_numpy(counts).to(DEV)
    rc = _lib.lib().stac_scores_update(ptr(torch.from_numpy(colsum).to(DEV)), T_live, ptr(d_s), ptr(d_c), Tb, H,
                                       T_live, old_T, Tq, 0.9, stream_ptr())
    assert rc == 0
    assert np.array_equal(d_s.cpu().numpy(), ref_s)
    assert np.array_equal(d_c.cpu().numpy(), ref_c)
    # compaction
    n_keep = 260
    keep = np.stack([np.sort(rs.choice(T_live, n_keep, replace=False)) for _ in range(H)]).astype(np.int32)
    K = torch.from_numpy(rs.randn(H, Tb, D).astype(np.float32)).to(torch.bfloat16).to(DEV)
    V = torch.from_numpy(rs.randn(H, Tb, D).astype(np.float32)).to(torch.bfloat16).to(DEV)
    TI = torch.from_numpy(rs.randint(0, 10 ** 6, size=(H, Tb)).astype(np.int64)).to(DEV)
    VX = torch.from_numpy(rs.randint(-1, 99, size=(H, Tb)).astype(np.int32)).to(DEV)
    K2, V2, TI2, VX2 = torch.zeros_like(K), torch.zeros_like(V), torch.zeros_like(TI), torch.zeros_like(VX)
    S2, C2 = torch.ones_like(d_s), torch.ones_like(d_c)
    rc = _lib.lib().stac_compact(ptr(torch.from_numpy(keep).to(DEV)), H, n_keep, Tb, D, 2, ptr(K), ptr(V), ptr(K2),
                                 ptr(V2), ptr(TI), ptr(TI2), ptr(d_s), ptr(S2), ptr(d_c), ptr(C2), ptr(VX), ptr(VX2),
                                 stream_ptr())
    assert rc == 0
    kk = torch.from_numpy(keep).long().to(DEV)
    assert torch.equal(K2[:, :n_keep], torch.gather(K, 1, kk[..., None].expand(-1, -1, D)))
    assert torch.equal(V2[:, :n_keep], torch.gather(V, 1, kk[..., None].expand(-1, -1, D)))
    assert torch.equal(TI2[:, :n_keep], torch.gather(TI, 1, kk))
    assert torch.equal(S2[:, :n_keep], torch.gather(d_s, 1, kk))
    assert torch.equal(VX2[:, :n_keep], torch.gather(VX, 1, kk))
    assert bool((TI2[:, n_keep:] == -1).all()) and bool((VX2[:, n_keep:] == -1).all())
    assert bool((S2[:, n_keep:] == 0).all()) and bool((C2[:, n_keep:] == 0).all())


def _compare_pool(snap, m, tag, rtol, atol):
    sm = m.slot_map()
    for key in ("buf_offset", "buf_seg", "piv_offset", "piv_seg"):
        assert np.array_equal(snap[key], sm[key]), (tag, key)
    assert snap["buf_top"] == sm["buf_top"] and snap["piv_top"] == sm["piv_top"], tag
    assert np.array_equal(snap["buf_free"], sm["buf_free"]), (tag, "free list")
    hv, oK, oV, oS = m.overflow_arrays()
    assert np.array_equal(snap["over_hv"], hv), (tag, "overflow rows")
    d = m.dense()
    for f in ("piv_K", "piv_V", "piv_W", "piv_S", "piv_C", "buf_K", "buf_V", "buf_S"):
        np.testing.assert_allclose(snap[f], d[f], rtol=rtol, atol=atol, err_msg=f"{tag} {f}")
    np.testing.assert_allclose(snap["over_K"], oK, rtol=rtol, atol=atol)
    np.testing.assert_allclose(snap["over_S"], oS, rtol=rtol, atol=atol)


def _same_order_up_to_near_ties(idx_gpu, idx_ref, oracle, tag):
    """The retrieved (voxel, slot) order must be the oracle's.  The order is by pivot weight, and
    the weights themselves agree only to rounding (sums of exp() evaluated by different libraries),
    so two pivots whose weights differ in the last bits may change places: allowed only when the
    oracle's weights of the two entries agree to 4e-6 relative and both lists hold the same
    entries.  Returns the [H, R] mask of positions where the lists agree."""
    same = (idx_gpu == idx_ref).all(-1)
    if same.all():
        return same

    def weight(h, v, p):
        return float(oracle.piv.data["W"][int(oracle.piv.row_seg[h, v, p])])
    for h, i in zip(*np.nonzero(~same)):
        (vg, pg), (vo, po) = idx_gpu[h, i], idx_ref[h, i]
        assert vg >= 0 and vo >= 0, (tag, h, i)
        wg, wo = weight(h, vg, pg), weight(h, vo, po)
        assert abs(wg - wo) <= 4e-6 * abs(wo), (tag, h, i, wg, wo)
    for h in range(idx_gpu.shape[0]):
        assert sorted(map(tuple, idx_gpu[h].tolist())) == sorted(map(tuple, idx_ref[h].tolist())), (tag, h)
    return same


@pytest.mark.parametrize("name", list(cases.MERGER_GPU) + ["f32_d64"])
def test_merge_and_retrieve_match_oracle(name):
    from stac_b200 import ops
    from stac_b200.stac.merger import VoxelKVMerger
    c = cases.merger_config(name)
    tdt = torch.float32 if c["dtype"] == "f32" else torch.bfloat16
    # bf16 pools: values are compared after bf16 storage, so allow a few bf16 ulps of a unit value
    rtol, atol = (1e-3, 1e-5) if c["dtype"] == "f32" else (8e-3, 4e-3)
    st = ops.DeviceStatus(torch.device(DEV))
    g = VoxelKVMerger(c["H"], c["D"], init_voxels=c["init_voxels"], pivot_cap=c["P"], budget_cap=c["B"],
                      sim_thresh=c["sim"], replace_thresh=c["replace"], score_thresh=c["score"], dtype=tdt,
                      device=DEV, allocator="segment", seg_size=1, slab_cap=16, status=st)
    m = VoxelMerger(c["H"], c["D"], c["init_voxels"], c["P"], c["B"], c["sim"], c["replace"], c["score"],
                    c["dtype"])
    t = VoxelTable(c["voxel_size"])
    for step, (pts, K, V, S) in enumerate(cases.merger_inputs(name)):
        ids = t.upsert(quantize(pts, c["voxel_size"]))
        VX = np.broadcast_to(ids, (c["H"], ids.size)).copy()
        VX[:, cases.merger_invalid_mask(name, step, ids.size)] = -1
        if step == 2:
            VX[:] = -1          # a call without any valid token leaves everything untouched
        Kr, Vr = m.rnd(K), m.rnd(V)
        m.insert_and_merge(Kr, Vr, S, VX, t.num_voxels)
        g.insert_and_merge(torch.from_numpy(Kr).to(DEV), torch.from_numpy(Vr).to(DEV), torch.from_numpy(S).to(DEV),
                           None, torch.from_numpy(VX).to(DEV), t.num_voxels)
        st.raise_if_set(f"merge step {step}")
        _compare_pool(g.snapshot(), m, f"{name} step {step}", rtol, atol)
    info = g.info()
    assert info["buffer_pool_used"] == m.buf.used() and info["pivot_pool_used"] == m.piv.used()
    # retrieval: order of (voxel, slot) must be identical
    rs = np.random.RandomState(5)
    for R in (16, 200, 1000, 6000):
        nq = t.num_voxels if R == 6000 else min(t.num_voxels, 300)     # the widest block queries every voxel
        q = rs.randint(0, t.num_voxels, size=nq).astype(np.int64)
        Kg, Vg, Mg, Bg, Ig = g.retrieve(torch.from_numpy(q).to(DEV), True, R, want_idx=True)
        Ko, Vo, Mo, Bo, Io = m.retrieve(q, R, True)
        assert np.array_equal(Mg.cpu().numpy(), Mo), (name, R)
        same = _same_order_up_to_near_ties(Ig.cpu().numpy(), Io, m, (name, R))
        np.testing.assert_allclose(Kg.float().cpu().numpy()[same], Ko[same], rtol=rtol, atol=atol)
        np.testing.assert_allclose(Vg.float().cpu().numpy()[same], Vo[same], rtol=rtol, atol=atol)
        fin = np.isfinite(Bo)
        assert np.array_equal(np.isfinite(Bg.cpu().numpy()), fin)
        np.testing.assert_allclose(Bg.cpu().numpy()[fin & same], Bo[fin & same], rtol=1e-5, atol=1e-6)
    # unbounded mode (retrieve_size <= 0): width = #voxels * P, optionally followed by buffer tokens
    q = rs.randint(0, t.num_voxels, size=min(t.num_voxels, 40)).astype(np.int64)
    for rb in (False, True):
        Kg, Vg, Mg, Bg, Ig = g.retrieve(torch.from_numpy(q).to(DEV), rb, -1, want_idx=True)
        Ko, Vo, Mo, Bo, Io = m.retrieve(q, -1, rb)
        assert Kg.shape == Ko.shape, (name, rb)
        assert np.array_equal(Mg.cpu().numpy(), Mo) and np.array_equal(Ig.cpu().numpy(), Io), (name, rb)
        np.testing.assert_allclose(Kg.float().cpu().numpy(), Ko, rtol=rtol, atol=atol)
        np.testing.assert_allclose(Vg.float().cpu().numpy(), Vo, rtol=rtol, atol=atol)
        fin = np.isfinite(Bo)
        assert np.array_equal(np.isfinite(Bg.cpu().numpy()), fin)
        np.testing.assert_allclose(Bg.cpu().numpy()[fin], Bo[fin], rtol=1e-5, atol=1e-6)


def _full_size_run(steps, seed):
    """384 pool heads x 8328 evicted tokens per call (the pool-stress shape), bf16: tokens fall on
    1500 voxels, half of their keys cluster around a per-voxel direction so that similarity
    merges, full rows, pivot insertion and victim re-merges all happen."""
    from stac_b200 import ops
    from stac_b200.stac.merger import VoxelKVMerger
    H, D, Tn, NV = 384, 64, 8328, 1500
    st = ops.DeviceStatus(torch.device(DEV))
    g = VoxelKVMerger(H, D, init_voxels=NV, pivot_cap=4, budget_cap=8, sim_thresh=0.8, replace_thresh=0.8,
                      score_thresh=0.2, dtype=torch.bfloat16, device=DEV, status=st)
    gen = torch.Generator(device=DEV).manual_seed(seed)
    dirs = torch.randn((NV, D), generator=gen, device=DEV)
    n_valid = 0
    for _ in range(steps):
        vx = torch.randint(0, NV, (Tn,), generator=gen, device=DEV, dtype=torch.int32)
        vx[torch.rand(Tn, generator=gen, device=DEV) < 0.03] = -1
        near = (torch.rand(Tn, generator=gen, device=DEV) < 0.5).view(1, Tn, 1)
        noise = torch.randn((H, Tn, D), generator=gen, device=DEV)
        K = torch.where(near, dirs[vx.clamp(min=0).long()].unsqueeze(0) + 0.3 * noise, noise).to(torch.bfloat16)
        V = torch.randn((H, Tn, D), generator=gen, device=DEV).to(torch.bfloat16)
        S = torch.rand((H, Tn), generator=gen, device=DEV)
        g.insert_and_merge(K, V, S, None, vx.view(1, Tn).expand(H, Tn).contiguous(), NV)
        n_valid += H * int((vx >= 0).sum())
        del K, V, S, noise
    st.raise_if_set("full-size merge")
    return g, n_valid


def test_full_size_voxel_memory_properties():
    """Properties that do not depend on the size, checked at the pool-stress size: no segment is
    handed out twice, rows stay inside their caps, buffered scores of a row are stored in rank
    order, no token is counted twice, retrieval returns distinct pivots in weight order, and
    a second run of the same stream ends in the same bits."""
    g, n_valid = _full_size_run(6, seed=7)
    H, P, B = g.H, g.P, g.B
    pc, bc = g._piv_row_cnt.long(), g._buf_row_cnt.long()
    assert int(pc.min()) >= 0 and int(pc.max()) <= P and int(bc.min()) >= 0 and int(bc.max()) <= B
    info = g.info()
    for cnt, seg, used in ((pc, g._piv_row_seg, info["pivot_pool_used"]), (bc, g._buf_row_seg, info["buffer_pool_used"])):
        live = torch.arange(seg.shape[2], device=DEV).view(1, 1, -1) < cnt.unsqueeze(-1)
        ids = seg[live]
        assert int(ids.numel()) == used and int(ids.min()) >= 0
        assert int(torch.unique(ids).numel()) == used            # every live segment belongs to one (row, column)
    assert int(pc.sum()) > 100000 and int((pc == P).sum()) > 0   # pivots formed, some rows saturated
    # buffered scores of a row: descending with the column
    sc = g._buf_S[g._buf_row_seg.clamp(min=0).long()]
    col = torch.arange(B, device=DEV).view(1, 1, B)
    both = (col[..., 1:] < bc.unsqueeze(-1))
    assert bool(((sc[..., :-1] >= sc[..., 1:]) | ~both).all())
    # tokens: pivots count what they absorbed, the rest is buffered, carried over or fell to the score gate
    live_p = torch.arange(P, device=DEV).view(1, 1, P) < pc.unsqueeze(-1)
    absorbed = float(g._piv_C[g._piv_row_seg[live_p].long()].double().sum())
    assert absorbed + info["buffer_pool_used"] <= n_valid and absorbed > 0.1 * n_valid
    # retrieval around every voxel: distinct pivots, weights descending, as many as there are (up to R)
    R = 2048
    K, V, M, Bz, I = g.retrieve(None, True, R, want_idx=True)
    n_piv = pc.sum(dim=1)
    assert torch.equal(M.sum(dim=1), torch.clamp(n_piv, max=R))
    w = g._piv_W[g._piv_row_seg[torch.arange(H, device=DEV).view(H, 1), I[..., 0].clamp(min=0).long(),
                                I[..., 1].clamp(min=0).long()].clamp(min=0).long()]
    ok = M[:, 1:] & M[:, :-1]
    assert bool(((w[:, :-1] >= w[:, 1:]) | ~ok).all())
    flat = (I[..., 0].long() * P + I[..., 1].long())
    for h in (0, 191, 383):
        sel = flat[h][M[h]]
        assert int(torch.unique(sel).numel()) == int(sel.numel())
    cnt_sel = g._piv_C[g._piv_row_seg[torch.arange(H, device=DEV).view(H, 1), I[..., 0].clamp(min=0).long(),
                                      I[..., 1].clamp(min=0).long()].clamp(min=0).long()]
    assert torch.allclose(Bz[M], torch.log(cnt_sel[M].clamp(min=1e-9)), rtol=1e-6, atol=1e-6)
    assert bool(torch.isinf(Bz[~M]).all())
    # same stream again: same bits
    g2, _ = _full_size_run(6, seed=7)
    for name in ("_piv_row_cnt", "_piv_row_seg", "_buf_row_cnt", "_buf_row_seg"):
        assert torch.equal(getattr(g, name), getattr(g2, name)), name
    n_p, n_b = info["pivot_pool_used"], info["buffer_pool_used"]
    for name in ("_piv_K", "_piv_V", "_piv_W", "_piv_S", "_piv_C"):
        a, b = getattr(g, name), getattr(g2, name)
        assert torch.equal(a[g._piv_row_seg[live_p].long()], b[g2._piv_row_seg[live_p].long()]), name
    del g2


def test_merge_is_deterministic():
    """Two pools fed the same stream end in bit-identical state (no atomics on values or slots)."""
    from stac_b200.stac.merger import VoxelKVMerger
    c = cases.merger_config("gpu_bf16")
    snaps = []
    for _ in range(2):
        g = VoxelKVMerger(c["H"], c["D"], init_voxels=64, pivot_cap=4, budget_cap=8, sim_thresh=0.8,
                          replace_thresh=0.8, score_thresh=0.2, dtype=torch.bfloat16, device=DEV)
        t = VoxelTable(0.05)
        for pts, K, V, S in cases.merger_inputs("gpu_bf16"):
            ids = t.upsert(quantize(pts, 0.05))
            VX = np.broadcast_to(ids, (c["H"], ids.size)).copy()
            g.insert_and_merge(torch.from_numpy(K).to(DEV), torch.from_numpy(V).to(DEV),
                               torch.from_numpy(S).to(DEV), None, torch.from_numpy(VX).to(DEV), t.num_voxels)
        snaps.append(g.snapshot())
    for k in snaps[0]:
        assert np.array_equal(np.asarray(snaps[0][k]), np.asarray(snaps[1][k])), k


@pytest.mark.parametrize("max_buf,max_piv", [(2500, None), (None, 150), (1800, 120)])
def test_bounded_pools_match_oracle(max_buf, max_piv):
    """With a bound on the segment pools, rows are skipped in (head, voxel) order once the pool
    is full; state and drop counts must match the oracle's statement of the same rule."""
    from stac_b200 import ops
    from stac_b200.stac.merger import VoxelKVMerger
    name = "gpu_f32"
    c = cases.merger_config(name)
    st = ops.DeviceStatus(torch.device(DEV))
    g = VoxelKVMerger(c["H"], c["D"], init_voxels=c["init_voxels"], pivot_cap=c["P"], budget_cap=c["B"],
                      sim_thresh=c["sim"], replace_thresh=c["replace"], score_thresh=c["score"], dtype=torch.float32,
                      device=DEV, slab_cap=16, status=st, max_buffer_slots=max_buf, max_pivot_slots=max_piv)
    m = VoxelMerger(c["H"], c["D"], c["init_voxels"], c["P"], c["B"], c["sim"], c["replace"], c["score"], "f32",
                    max_buf_slots=max_buf, max_piv_slots=max_piv)
    t = VoxelTable(c["voxel_size"])
    for step, (pts, K, V, S) in enumerate(cases.merger_inputs(name)):
        ids = t.upsert(quantize(pts, c["voxel_size"]))
        VX = np.broadcast_to(ids, (c["H"], ids.size)).copy()
        m.insert_and_merge(K, V, S, VX, t.num_voxels)
        g.insert_and_merge(torch.from_numpy(K).to(DEV), torch.from_numpy(V).to(DEV), torch.from_numpy(S).to(DEV),
                           None, torch.from_numpy(VX).to(DEV), t.num_voxels)
        st.raise_if_set(f"bounded merge step {step}")
        _compare_pool(g.snapshot(), m, f"bounded step {step}", 1e-3, 1e-5)
        assert g.info()["dropped_tokens"] == m.dropped, step
        if max_buf is not None:
            assert g.snapshot()["buf_top"] <= max_buf
        if max_piv is not None:
            assert g.snapshot()["piv_top"] <= max_piv
    assert m.dropped > 0
