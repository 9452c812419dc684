"""The CPU oracle against the fixtures produced by the reference's own Python path
(tests/golden/make_golden.py).  Integer outputs must be identical; merged values within
1e-3 relative (fp32 arithmetic in a different summation order)."""

import os

import numpy as np
import pytest

import cases
from oracle.attention import attn_colsum, subsample_plan
from oracle.manager import StacManager
from oracle.pool import VoxelMerger
from oracle.voxel import VoxelTable, pack_keys, quantize

INT_KEYS = ("buf_state", "buf_offset", "buf_seg", "piv_state", "piv_offset", "piv_seg",
            "buf_top", "piv_top", "buf_free")


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def _close(a, b, rtol=1e-3, atol=1e-5):
    np.testing.assert_allclose(a, b, rtol=rtol, atol=atol)


def test_voxel_table(golden_dir):
    g = _load(golden_dir, "voxel_table.npz")
    c = cases.VOXEL
    t = VoxelTable(c["voxel_size"])
    for step, pts in enumerate(cases.voxel_points()):
        ijk = quantize(pts, c["voxel_size"])
        assert np.array_equal(ijk, g[f"ijk_{step}"])
        ids = t.upsert(ijk)
        assert np.array_equal(ids, g[f"ids_{step}"])
        nb = t.neighbors(g[f"query_{step}"], R=2)
        assert np.array_equal(nb, g[f"nbr_{step}"])
    assert np.array_equal(t.keys, g["keys_1d"])
    assert np.array_equal(t.ijk, g["table_ijk"])
    assert np.array_equal(pack_keys(t.ijk), t.keys)


def _check_slot_map(m, g, prefix):
    sm = m.slot_map()
    for k in INT_KEYS:
        ref = g[f"{prefix}_{k}"]
        got = np.asarray(sm[k])
        assert np.array_equal(got.astype(np.int64).reshape(ref.shape), ref.astype(np.int64)), (prefix, k)
    hv, _, _, _ = m.overflow_arrays()
    assert np.array_equal(hv, g[f"{prefix}_over_hv"]), (prefix, "overflow rows")


@pytest.mark.parametrize("name", list(cases.MERGER))
def test_merger(golden_dir, name):
    g = _load(golden_dir, f"merger_{name}.npz")
    c = cases.MERGER[name]
    t = VoxelTable(c["voxel_size"])
    m = VoxelMerger(c["H"], c["D"], c["init_voxels"], c["P"], c["B"], c["sim"], c["replace"],
                    c["score"], c["dtype"])
    rtol = 1e-3 if c["dtype"] == "f32" else 1.6e-2
    for step, (pts, K, V, S) in enumerate(cases.merger_inputs(name)):
        ids = t.upsert(quantize(pts, c["voxel_size"]))
        VX = np.broadcast_to(ids, (c["H"], ids.size)).copy()
        VX[:, cases.merger_invalid_mask(name, step, ids.size)] = -1
        m.insert_and_merge(m.rnd(K), m.rnd(V), S, VX, t.num_voxels)
        assert t.num_voxels == int(g[f"s{step}_V"])
        _check_slot_map(m, g, f"s{step}")
        if step in c["dump_steps"]:
            d = m.dense()
            for f in ("piv_K", "piv_V", "piv_W", "piv_S", "piv_C", "buf_K", "buf_V", "buf_S"):
                _close(d[f], g[f"s{step}_{f}"], rtol=rtol, atol=rtol * 1e-1)
            _, oK, oV, oS = m.overflow_arrays()
            _close(oK, g[f"s{step}_over_K"], rtol=rtol)
            _close(oS, g[f"s{step}_over_S"], rtol=rtol)
    for tag, (q, R, rb) in c["retrieve"].items():
        qs = None if q is None else cases.retrieve_query(name, tag)
        Kr, Vr, Mr, Br, _ = m.retrieve(qs, R, rb)
        assert np.array_equal(Mr, g[f"ret_{tag}_M"]), tag
        assert Kr.shape == g[f"ret_{tag}_K"].shape
        _close(Kr, g[f"ret_{tag}_K"], rtol=rtol, atol=rtol * 1e-1)
        _close(Vr, g[f"ret_{tag}_V"], rtol=rtol, atol=rtol * 1e-1)
        fin = np.isfinite(g[f"ret_{tag}_B"])
        assert np.array_equal(np.isfinite(Br), fin)
        _close(Br[fin], g[f"ret_{tag}_B"][fin], rtol=1e-5)


def test_manager_trace(golden_dir):
    g = _load(golden_dir, "manager_trace.npz")
    c = cases.MANAGER
    mg = StacManager(c["L"], c["H"], c["D"], c["tpf"], c["buffer"], chunk_size=c["chunk"],
                     recent_size=c["window"], pinned_idx=(0,), hh_size=c["hh"], temperature=0.9,
                     voxel_size=c["voxel_size"], init_voxels=c["init_voxels"],
                     retrieval_size=c["retrieval"], dtype="f32")
    pruned = 0
    valid_pivots = 0      # retrieved pivots with a finite bias (log C) in the reference's own trace
    for step, (k, v, cs, pts, mask) in enumerate(cases.manager_inputs()):
        Tq = k.shape[2]
        for l in range(c["L"]):
            mg.append_kv(k[l], v[l], l)
            mg.update_scores(cs[l][:, : mg.off[l]], l, Tq)
        mg.append_positions(pts, mask)
        rec = np.empty(0, np.int64) if mg.recent_ids is None else np.unique(mg.recent_ids)
        assert np.array_equal(rec, g[f"s{step}_recent"]), step
        if step in c["retrieve_steps"]:
            mg.ret = None
            mg.retrieve(return_buf=True)
            T_ret = g[f"s{step}_ret_T"]
            if T_ret[0] > 0:
                Kr, _, Br, _, _ = mg.ret
                L, H = c["L"], c["H"]
                _close(Kr.reshape(L, H, -1, c["D"]), g[f"s{step}_ret_K"])
                refb = g[f"s{step}_ret_bias"]
                fin = np.isfinite(refb)
                valid_pivots += int(fin.sum())
                assert np.array_equal(np.isfinite(Br.reshape(refb.shape)), fin)
                _close(Br.reshape(refb.shape)[fin], refb[fin], rtol=1e-5)
        mg.prune()
        T = int(g[f"s{step}_T"])
        assert mg.off[0] == T
        pruned += mg.last_keep is not None
        assert np.array_equal(mg.TI[:, :, :T], g[f"s{step}_TI"]), step
        assert np.array_equal(mg.VX[:, :, :T], g[f"s{step}_VX"]), step
        _close(mg.S[:, :, :T], g[f"s{step}_S"], rtol=1e-6)
        assert mg.merger.V_used == int(g[f"s{step}_Vused"])
        _check_slot_map(mg.merger, g, f"s{step}")
    assert pruned >= 8
    # the trace must reach the states that matter: rows that filled up and became pivots, and
    # retrievals that returned them (log C hand-off, width rule of stac/stac_voxel.py:722-738)
    assert valid_pivots >= 300
    assert (g[f"s{c['steps'] - 1}_piv_offset"] > 0).sum() >= 100
    _close(mg.K[:, :, : mg.off[0]], g["final_K"], rtol=0, atol=0)


@pytest.mark.parametrize("name", list(cases.ATTENTION))
def test_attention(golden_dir, name):
    g = _load(golden_dir, "attention.npz")
    q, k, v, bias = cases.attention_inputs(name)
    out, lse, cs = attn_colsum(q, k, v, bias)
    _close(out, g[f"{name}_out"], rtol=1e-4, atol=1e-5)
    _close(lse, g[f"{name}_lse"], rtol=1e-5, atol=1e-5)
    _close(cs, g[f"{name}_colsum"], rtol=1e-4, atol=1e-6)
    _close(cs.sum(axis=1), np.full(cs.shape[0], q.shape[0], np.float32), rtol=1e-4)


def _bf16_bits_to_f32(a):
    return (a.view(np.uint16).astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("name", list(cases.ATTENTION_REF))
def test_attention_against_the_reference_kernels(golden_dir, name):
    """attention_ref.npz holds what the reference's own Triton kernels (fa_forward_colsum_fast_sub,
    stac/flash_attn_triton.py:900-1006) returned on a B200 for these seeded inputs
    (make_attention_ref.py).  The oracle, using that entry point's row sub-sampling rule, must
    reproduce O, lse and the column sums."""
    g = _load(golden_dir, "attention_ref.npz")
    c = cases.ATTENTION_REF[name]
    q, k, v, bias = cases.attention_inputs(name)
    out, lse, cs = attn_colsum(q, k, v, bias, subsample_ratio=c["ratio"], rule="triton")
    assert np.abs(out - _bf16_bits_to_f32(g[f"{name}_out_bf16"])).max() <= 2e-2      # bf16 output
    _close(lse, g[f"{name}_lse"], rtol=1e-3, atol=1e-3)
    _close(cs, g[f"{name}_colsum"], rtol=1e-3, atol=1e-6)
    if c["same_rule"]:   # both backends of the reference define the column sums identically here
        _, _, cs_cuda = attn_colsum(q, k, v, bias, subsample_ratio=c["ratio"])
        _close(cs_cuda, g[f"{name}_colsum"], rtol=1e-3, atol=1e-6)


def test_subsample_plan():
    assert subsample_plan(1041, 1.0) == (1041, 1, 1.0)
    assert subsample_plan(4164, 0.25) == (1024, 4, 4164 / 1024)
    assert subsample_plan(100, 0.25) == (100, 1, 1.0)
    assert subsample_plan(1041, 0.999) == (1024, 1, 1041 / 1024)
    assert subsample_plan(4164, 0.5) == (2048, 2, 4164 / 2048)
    # the Triton entry point has no exact special case at ratio 1
    assert subsample_plan(1041, 1.0, rule="triton") == (1024, 1, 1041 / 1024)
    assert subsample_plan(1024, 1.0, rule="triton") == (1024, 1, 1.0)


@pytest.mark.parametrize("name", list(cases.POINTMAP))
def test_pointmap(golden_dir, name):
    """Patch points and masks against StreamSession.get_pointmap run on CPU: bit-identical at the
    production frame size (all weights 1/4), one unit in the last place at a ragged size."""
    from oracle.pointmap import pointmap_to_positions
    g = _load(golden_dir, "pointmap.npz")
    c = cases.POINTMAP[name]
    wp, cf = cases.pointmap_inputs(name)
    pts, mask = pointmap_to_positions(wp, cf, c["patch"], c["conf_threshold"], c["special"])
    assert np.array_equal(mask, g[f"{name}_mask"])
    if name == "frame":
        assert np.array_equal(pts, g[f"{name}_pts"])
    else:
        np.testing.assert_allclose(pts, g[f"{name}_pts"], rtol=4e-6, atol=1e-7)
    assert mask[:, :c["special"]].sum() == 0 and np.all(pts[:, :c["special"]] == 0)
