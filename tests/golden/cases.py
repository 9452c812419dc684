"""Seeded input generators shared by ``make_golden.py`` (which feeds them to the reference)
and by the tests (which feed them to the oracle and to the CUDA path)."""

import numpy as np

# ---------------------------------------------------------------- voxel table
VOXEL = {"voxel_size": 0.05, "steps": 4, "n_points": 600, "n_query": 64, "seed": 11}


def voxel_points():
    rs = np.random.RandomState(VOXEL["seed"])
    prev = None
    for step in range(VOXEL["steps"]):
        pts = (rs.rand(VOXEL["n_points"], 3).astype(np.float32) - 0.5) * np.float32(1.2)
        if prev is not None:
            pts[:200] = prev[100:300]          # revisit known voxels
            pts[200:230] = pts[230:260]        # duplicates inside one call
        pts[-3:] = np.array([[0.05, -0.05, 0.1], [0.0, 0.0, 0.0], [-0.15, 0.2, -0.05]], np.float32)
        prev = pts
        yield pts


# ---------------------------------------------------------------- merger
_M = dict(P=4, B=8, sim=0.8, replace=0.8, score=0.2, voxel_size=0.05)
MERGER = {
    "f32_small": dict(_M, H=3, D=16, N=512, steps=12, init_voxels=16, dtype="f32", seed=21,
                      n_sites=40, dump_steps=(3, 7, 11),
                      retrieve={"bounded": ("q", 64, True), "unbounded_buf": ("q", -1, True),
                                "all": (None, None, False)}),
    "bf16_small": dict(_M, H=3, D=16, N=512, steps=12, init_voxels=16, dtype="bf16", seed=22,
                       n_sites=40, dump_steps=(3, 7, 11),
                       retrieve={"bounded": ("q", 64, True), "all": (None, None, False)}),
    "f32_d64": dict(_M, H=2, D=64, N=384, steps=8, init_voxels=64, dtype="f32", seed=23,
                    n_sites=24, dump_steps=(7,),
                    retrieve={"bounded": ("q", 48, False)}),
}


# GPU-vs-oracle cases (no reference fixture needed: the oracle is pinned by the cases above)
MERGER_GPU = {
    "gpu_f32": dict(_M, H=4, D=64, N=1536, steps=10, init_voxels=32, dtype="f32", seed=51, n_sites=96),
    "gpu_bf16": dict(_M, H=4, D=64, N=1536, steps=10, init_voxels=32, dtype="bf16", seed=52, n_sites=96),
    "gpu_wide": dict(_M, H=6, D=64, N=4000, steps=4, init_voxels=4096, dtype="bf16", seed=53, n_sites=2500),
    "gpu_crowded": dict(_M, H=2, D=64, N=3000, steps=5, init_voxels=8, dtype="f32", seed=54, n_sites=3),
    # more than 8192 tokens per pool head and call: the per-head sort leaves its register path
    "gpu_long": dict(_M, H=2, D=64, N=9100, steps=3, init_voxels=1024, dtype="bf16", seed=55, n_sites=1500),
}


def merger_config(name):
    return MERGER[name] if name in MERGER else MERGER_GPU[name]


def merger_inputs(name):
    """Yields (points [N,3], K [H,N,D], V [H,N,D], S [H,N]) per step.  Points visit a slowly
    growing set of sites so that buffers fill, pivots appear, saturate and get re-merged;
    part of the keys cluster around a per-site direction so the similarity merge triggers."""
    c = merger_config(name)
    rs = np.random.RandomState(c["seed"])
    H, D, N = c["H"], c["D"], c["N"]
    sites = (rs.rand(c["n_sites"] * 3, 3).astype(np.float32) - 0.5) * np.float32(1.5)
    dirs = rs.randn(c["n_sites"] * 3, H, D).astype(np.float32)
    for step in range(c["steps"]):
        n_live = min(sites.shape[0], c["n_sites"] + 6 * step)
        which = rs.randint(0, n_live, size=N)
        pts = sites[which] + (rs.rand(N, 3).astype(np.float32) - 0.5) * np.float32(0.01)
        noise = rs.randn(H, N, D).astype(np.float32)
        near = rs.rand(N) < 0.5
        K = np.where(near[None, :, None], dirs[which].transpose(1, 0, 2) + np.float32(0.3) * noise, noise)
        V = rs.randn(H, N, D).astype(np.float32)
        S = rs.rand(H, N).astype(np.float32)
        yield pts.astype(np.float32), K.astype(np.float32), V, S


def merger_invalid_mask(name, step, N):
    rs = np.random.RandomState(1000 + step)
    if step % 3 == 0:
        return rs.rand(N) < 0.05
    return np.zeros(N, bool)


def retrieve_query(name, tag):
    rs = np.random.RandomState(77)
    return rs.randint(0, 60, size=40).astype(np.int64)


# ---------------------------------------------------------------- manager trace
# `motion` = camera shift per frame (m): slow enough that a voxel is seen in many frames, so buffer
# rows fill up, pivots form and the retrieval around the newest frames returns valid pivots.
MANAGER = dict(L=2, H=2, D=16, tpf=21, special=5, chunk=2, window=3, hh=1, buffer=7, steps=24,
               voxel_size=0.05, init_voxels=32, retrieval=1, retrieve_steps=(6, 10, 14, 16, 18, 20, 22),
               seed=31, motion=0.003)


MANAGER_GPU = dict(L=2, H=3, D=64, tpf=41, special=5, chunk=2, window=3, hh=1, buffer=7, steps=26,
                   voxel_size=0.05, init_voxels=32, retrieval=1, retrieve_steps=(6, 8, 10, 12, 14, 16, 18, 20, 22, 24),
                   seed=61, motion=0.003)


def manager_inputs(c=None):
    """Yields per chunk: k, v [L,H,Tn,D], column sums [L,H,T_buf], points [Tn,3], mask [Tn]."""
    c = MANAGER if c is None else c
    rs = np.random.RandomState(c["seed"])
    L, H, D, tpf = c["L"], c["H"], c["D"], c["tpf"]
    Tn = c["chunk"] * tpf
    T_buf = c["buffer"] * tpf
    npatch = tpf - c["special"]
    side = int(round(npatch ** 0.5))
    gx, gy = np.meshgrid(np.arange(side), np.arange(side), indexing="ij")
    grid = np.stack([gx.reshape(-1), gy.reshape(-1), np.zeros(side * side)], 1).astype(np.float32)
    for step in range(c["steps"]):
        k = rs.randn(L, H, Tn, D).astype(np.float32)
        v = rs.randn(L, H, Tn, D).astype(np.float32)
        cs = (rs.rand(L, H, T_buf).astype(np.float32) + np.float32(0.01))
        pts = np.zeros((Tn, 3), np.float32)
        mask = np.zeros(Tn, bool)
        for f in range(c["chunk"]):
            frame = step * c["chunk"] + f
            p = grid * np.float32(0.06) + np.array([c.get("motion", 0.02) * frame, 0.0, 0.3], np.float32)
            p = p + (rs.rand(npatch, 3).astype(np.float32) - 0.5) * np.float32(0.02)
            lo = f * tpf + c["special"]
            pts[lo:lo + npatch] = p
            mask[lo:lo + npatch] = rs.rand(npatch) < 0.9
        yield k, v, cs, pts, mask


# ---------------------------------------------------------------- attention
ATTENTION = {
    "plain": dict(M=70, N=200, H=2, D=64, n_bias=0, seed=41),
    "pivots": dict(M=130, N=300, H=2, D=64, n_bias=64, seed=42),
}


# Cases run through the reference's own Triton kernels on a B200 (make_attention_ref.py).
# "ratio" is the subsample_ratio passed; where M is not a multiple of 128 the Triton entry
# point sums rows [0, M//128*128) and rescales even at ratio 1 (the CUDA backend, which the
# library follows, is exact there), so "same_rule" says whether the column sums of the two
# backends are defined identically for the case.
ATTENTION_REF = {
    "plain": dict(M=70, N=200, H=2, D=64, n_bias=0, seed=41, ratio=1.0, same_rule=True),
    "pivots": dict(M=130, N=300, H=2, D=64, n_bias=64, seed=42, ratio=1.0, same_rule=False),
    "pivots256": dict(M=256, N=700, H=3, D=64, n_bias=190, seed=43, ratio=1.0, same_rule=True),
    "subsample": dict(M=512, N=900, H=2, D=64, n_bias=130, seed=44, ratio=0.25, same_rule=True),
    "config2_tail": dict(M=1024, N=2082, H=4, D=64, n_bias=2048, seed=45, ratio=1.0, same_rule=True),
    "config2_frame": dict(M=1041, N=2082, H=2, D=64, n_bias=2048, seed=46, ratio=1.0, same_rule=False),
}


def attention_inputs(name):
    """q [M,H,D], k/v [N,H,D] float32 holding bf16-representable values, bias [H,N] or None."""
    c = ATTENTION[name] if name in ATTENTION else ATTENTION_REF[name]
    rs = np.random.RandomState(c["seed"])

    def bf16(x):
        u = x.astype(np.float32).view(np.uint32)
        return ((u + 0x8000) & 0xFFFF0000).astype(np.uint32).view(np.float32)

    q = bf16(rs.randn(c["M"], c["H"], c["D"]) / 8 * 6)
    k = bf16(rs.randn(c["N"], c["H"], c["D"]) / 8 * 6)
    v = bf16(rs.randn(c["N"], c["H"], c["D"]) / 8)
    bias = None
    if c["n_bias"]:
        bias = np.zeros((c["H"], c["N"]), np.float32)
        cnt = rs.randint(1, 9, size=(c["H"], c["n_bias"])).astype(np.float32)
        b = np.log(cnt)
        b[rs.rand(c["H"], c["n_bias"]) < 0.25] = -np.inf
        bias[:, c["N"] - c["n_bias"]:] = b
    return q, k, v, bias


# ---------------------------------------------------------------- point map -> patch points
# "frame" is the production shape (518 x 392, 14-pixel patches, 5 special tokens per frame);
# "ragged" is not a multiple of the patch (weights other than 1/4).
POINTMAP = {
    "frame": dict(S=2, H=392, W=518, patch=14, special=5, conf_threshold=1.0, seed=51),
    "ragged": dict(S=3, H=45, W=61, patch=14, special=2, conf_threshold=1.5, seed=52),
}


def pointmap_inputs(name):
    """world points f32 [S,H,W,3] (a smooth surface plus noise, metres) and confidence [S,H,W]."""
    c = POINTMAP[name]
    rs = np.random.RandomState(c["seed"])
    S, H, W = c["S"], c["H"], c["W"]
    yy, xx = np.meshgrid(np.linspace(-1, 1, H), np.linspace(-1, 1, W), indexing="ij")
    depth = 3.0 + np.sin(2.0 * xx)[None] + 0.5 * np.cos(3.0 * yy)[None] + 0.3 * np.arange(S)[:, None, None]
    pts = np.stack([xx[None] * depth, yy[None] * depth, depth], axis=-1) + rs.randn(S, H, W, 3) * 0.01
    conf = 0.2 + 2.0 * rs.rand(S, 1, 1) * (0.5 + 0.5 * np.cos(4.0 * xx + yy)[None]) + rs.rand(S, H, W) * 1.2
    return pts.astype(np.float32), conf.astype(np.float32)
