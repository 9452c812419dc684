"""Run the reference's own ``StreamSession.pipeline`` (stream_session.py:258-565), unchanged, on
a random-init ``CausalVGGT`` with either this library's managers or the reference's own.

    python tests/stream_session_run.py --manager stac_b200 --model tiny --frames 32
    python tests/stream_session_run.py --manager reference --model full --frames 300

``--manager stac_b200`` registers ``stac_b200.stac`` under the module name ``stac`` before the
reference's modules are imported (``stac_b200.compat.install_as_stac``), so every
``from stac... import`` in the reference's callers binds this library; nothing else is
patched.  ``--manager reference`` imports the reference's ``stac`` package from ``oracle/_ref``
(Triton attention, Python voxel path: the backends that need no compiled extension).
``--model full`` is the architecture of the end-to-end configuration (24-layer ViT-L
aggregator, dim 1024, 16 heads, camera head, two DPT heads, 518x392 frames); ``tiny`` keeps the
24 layers and head_dim 64 with the ViT-S embed (dim 384, 6 heads) and small heads, on 56x70
frames, so that a test finishes in seconds.
Weights are random and frames are seeded uniform noise: no dataset item is used.  With random
weights the predicted confidences and points are arbitrary, so the confidence threshold is
lowered to 1.0 (confidence = 1 + exp(x) > 1 always) and, unless given, the voxel size is
chosen from the spread of the points predicted for the first frame (about 24 cells across the
central 90 % of the widest axis), so that tokens spread over voxels as they do in a real scene.

Prints one JSON line.  Test infrastructure: needs ``oracle/_ref`` (python oracle/make_ref.py).
"""

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def build_model(kind, torch):
    from causalvggt.heads.camera_head import CameraHead
    from causalvggt.heads.dpt_head import DPTHead
    from causalvggt.models.aggregator import CausalAggregator
    from causalvggt.models.vggt import CausalVGGT
    torch.manual_seed(0)
    if kind == "full":
        return CausalVGGT(img_size=518, patch_size=14, embed_dim=1024)
    # same class, small widths: the constructor hard-wires the ViT-L sizes, so fill the fields
    m = CausalVGGT.__new__(CausalVGGT)
    torch.nn.Module.__init__(m)
    # (the smallest DINOv2 embed: StreamSession reads an integer patch size from it, which the
    # plain convolutional embed does not have)
    dim = 384
    m.aggregator = CausalAggregator(img_size=518, patch_size=14, embed_dim=dim, depth=24, num_heads=6,
                                    patch_embed="dinov2_vits14_reg")
    m.camera_head = CameraHead(dim_in=2 * dim, trunk_depth=2, num_heads=4)
    small = dict(features=32, out_channels=[32, 64, 128, 128])
    m.point_head = DPTHead(dim_in=2 * dim, output_dim=4, activation="inv_log", conf_activation="expp1", **small)
    m.depth_head = DPTHead(dim_in=2 * dim, output_dim=2, activation="exp", conf_activation="expp1", **small)
    m.track_head = None
    m.enable_camera, m.enable_point, m.enable_depth, m.enable_track = True, True, True, False
    return m


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--manager", choices=["stac_b200", "reference"], required=True)
    ap.add_argument("--model", choices=["tiny", "full"], default="tiny")
    ap.add_argument("--frames", type=int, default=32)
    ap.add_argument("--height", type=int, default=0)
    ap.add_argument("--width", type=int, default=0)
    ap.add_argument("--voxel-size", type=float, default=0.0)
    ap.add_argument("--dump", default="")
    args = ap.parse_args()
    if not os.path.isfile(os.path.join(REF, "stream_session.py")):
        sys.exit("oracle/_ref is missing: run `python oracle/make_ref.py /path/to/reference`")
    sys.path.insert(0, ROOT)
    import torch
    if args.manager == "stac_b200":
        from stac_b200.compat import install_as_stac
        install_as_stac()
    sys.path.insert(0, REF)        # causalvggt, stream_session (and the reference's stac unless aliased)
    import logging
    logging.disable(logging.INFO)
    from stream_session import StreamSession
    import stac.stac_voxel as bound
    H = args.height or (392 if args.model == "full" else 56)
    W = args.width or (518 if args.model == "full" else 70)
    dev = torch.device("cuda:0")
    model = build_model(args.model, torch).eval()
    g = torch.Generator().manual_seed(1)
    images = torch.rand(args.frames, 3, H, W, generator=g)
    session = StreamSession(model, device=dev)
    voxel_size = args.voxel_size
    if voxel_size <= 0:
        with torch.no_grad(), torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
            first = model(images=images[0:1].to(dev), mode="full", camera_head_kv_cache_list=None, streaming=True,
                          is_anchor_exist=True)
        pts = first["world_points"].float().reshape(-1, 3)
        lo, hi = torch.quantile(pts[::7], 0.05, dim=0), torch.quantile(pts[::7], 0.95, dim=0)
        voxel_size = max(float((hi - lo).max()) / 24.0, 1e-6)
        del first, pts
    # the `stac` preset (model_wrapper.py:86-115) with the backends that run without a build step
    kwargs = dict(window_size=4, chunk_size=4, hh_size=2, retrieval_size=2, return_buf=True,
                  temperature=0.9, attn_backend="triton", subsample_ratio=1.0, pinned_frame_indices=[0],
                  voxel_size=voxel_size, voxel_num=4096,
                  conf_threshold=1.0, voxel_buf_cap=8, voxel_piv_cap=4, voxel_backend="python",
                  allocator="segment")
    torch.cuda.synchronize()
    t0 = time.time()
    with torch.no_grad(), torch.amp.autocast(device_type="cuda", dtype=torch.bfloat16):
        session.pipeline(images, mode="window_chunk_merge", dtype=torch.bfloat16, device=dev, **kwargs)
    torch.cuda.synchronize()
    wall = time.time() - t0
    bm = session.get_benchmark()
    stage_ms = {k: float(v) / args.frames for k, v in bm.items()}
    total_ms = sum(stage_ms.values())
    mem = session.get_stats().get("Memory(MB)", {})
    merger_info = session.model.aggregator.kv_manager.get_merger_info()
    preds = session.get_all_predictions()
    finite = all(bool(torch.isfinite(v).all()) for v in preds.values() if isinstance(v, torch.Tensor))
    res = {
        "manager": args.manager, "manager_module": bound.__file__.replace(ROOT + "/", ""),
        "model": args.model, "frames": args.frames, "frame_hw": [H, W], "voxel_size": voxel_size,
        # the reference's own FPS definition (model_wrapper.py:131-138): 1000 / sum of per-frame stage ms
        "fps_stage_sum": 1000.0 / total_ms if total_ms > 0 else 0.0,
        "fps_wall": args.frames / wall, "wall_s": wall, "stage_ms_per_frame": stage_ms,
        "memory_keys": sorted(mem.keys()), "memory_mb": {k: float(v) for k, v in mem.items()},
        "processed_frames": int(preds["world_points"].shape[1]), "finite": finite,
        "merger_info": {k: (float(v) if isinstance(v, float) else int(v)) for k, v in merger_info.items()
                        if isinstance(v, (int, float))},
    }
    if args.dump:
        torch.save({k: v for k, v in preds.items() if isinstance(v, torch.Tensor)}, args.dump)
    session.clear()
    print(json.dumps(res))


if __name__ == "__main__":
    main()
