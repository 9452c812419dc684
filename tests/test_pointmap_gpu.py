"""Point maps -> patch points -> voxel ids on the GPU, through the C ABI, against the oracle and
the reference's own output (tests/golden/pointmap.npz)."""

import os

import numpy as np
import pytest
import torch

import cases
from oracle.pointmap import pointmap_to_positions as oracle_pointmap
from oracle.voxel import VoxelTable, quantize

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", list(cases.POINTMAP))
def test_pointmap_matches_oracle_and_reference(name, golden_dir):
    from stac_b200.stac.pointmap import pointmap_to_positions
    dev = torch.device("cuda:0")
    c = cases.POINTMAP[name]
    wp, cf = cases.pointmap_inputs(name)
    pts, mask = pointmap_to_positions(torch.from_numpy(wp)[None].to(dev), torch.from_numpy(cf)[None].to(dev),
                                      c["patch"], c["conf_threshold"], c["special"])
    torch.cuda.synchronize()
    pts, mask = pts.cpu().numpy(), mask.cpu().numpy()
    o_pts, o_mask = oracle_pointmap(wp, cf, c["patch"], c["conf_threshold"], c["special"])
    assert np.array_equal(pts, o_pts) and np.array_equal(mask, o_mask)        # same fp32 operations in the same order
    g = np.load(os.path.join(golden_dir, "pointmap.npz"))
    assert np.array_equal(mask, g[f"{name}_mask"])
    if name == "frame":
        assert np.array_equal(pts, g[f"{name}_pts"])


def test_append_pointmap_gives_the_voxel_ids_of_the_two_step_path():
    """STACVoxelKV.append_pointmap == get_pointmap followed by append_positions: same voxel ids
    as the oracle's table fed with the oracle's patch points."""
    from stac_b200.stac import STACVoxelKV
    dev = torch.device("cuda:0")
    c = cases.POINTMAP["frame"]
    wp, cf = cases.pointmap_inputs("frame")
    S = c["S"]
    tpf = c["special"] + (c["H"] // c["patch"]) * (c["W"] // c["patch"])
    L, H, D = 1, 2, 64
    kv = STACVoxelKV(num_layers=L, num_heads=H, head_dim=D, token_per_frame=tpf, buffer_size=S + 3, chunk_size=S,
                     recent_size=1, pinned_idx=[0], hh_size=1, temperature=0.9, device=dev, dtype=torch.bfloat16,
                     voxel_size=0.05, init_voxels=64, voxel_buf_cap=8, voxel_piv_cap=4, retrieval_size=1)
    kv.reset()
    k = torch.zeros(1, H, S * tpf, D, dtype=torch.bfloat16, device=dev)
    kv.append_kv(k, k, 0)
    pts, mask = kv.append_pointmap(torch.from_numpy(wp)[None].to(dev), torch.from_numpy(cf)[None].to(dev),
                                   c["patch"], c["conf_threshold"], c["special"])
    torch.cuda.synchronize()
    o_pts, o_mask = oracle_pointmap(wp, cf, c["patch"], c["conf_threshold"], c["special"])
    table = VoxelTable()
    m = o_mask.reshape(-1)
    want = np.full(m.shape, -1, np.int32)
    want[m] = table.upsert(quantize(o_pts.reshape(-1, 3), 0.05)[m])
    got = kv._token_voxel_indices[0, 0, :S * tpf].cpu().numpy()
    assert np.array_equal(got, want)
    assert (got >= 0).sum() == m.sum() and got.max() + 1 == table.num_voxels
