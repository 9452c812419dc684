"""Benchmark of the STAC KV-cache compression hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one chunk of the streaming loop through the hot path, in the reference's call
order (stream_session.py:451-553): for each of the 24 managed layers append_kv +
decode_sparse_attn (window + pivot attention with column sums -> H2O scores), then
append_positions (points -> voxel ids, neighbour query), retrieve_kv on the reference's
schedule, prune_kv (H2O selection, eviction merge into the voxel memory, compaction).
The CausalVGGT backbone is outside this path: its per-layer q/k/v activations are replaced by
seeded random bf16 tensors of the same shape and its point maps by a synthetic smooth depth
surface seen from a moving camera.

Prints ONE JSON line (see the keys below).  `value` is device-resident throughput; `e2e` runs
the same steps with q/k/v and points copied from pinned host memory (on a copy stream, one
step ahead of the compute, into two staging sets) and the last layer's output read back every
step.  With N > 1 every rank runs an independent stream (weak scaling,
no data-path collective); the timed region is bracketed by barriers and the maximum over
ranks is used.
"""

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(layers=24, heads=16, head_dim=64, tpf=1041, special=5, patch_h=37, patch_w=28, chunk=4, window=8,
           hh=2, pinned=[0], retrieval=2, voxel_size=0.05, init_voxels=4096, buf_cap=8, piv_cap=4,
           temperature=0.9, prefill_chunks=40,
           # bounded voxel memory of the long-stream configuration: 2M slots per layer
           max_buffer_slots=2_000_000 * 24, max_pivot_slots=2_000_000 * 24)
ATTN_TRAFFIC_BYTES_PER_CALL = 138.9e6
METRIC = "stac_hot_path_streaming_frames_per_sec"
WORKLOAD = ("config4-hot-path: CausalVGGT+STAC stream shapes (24 layers x 16 heads x 64, 1041 tokens/frame, "
            "chunk 4, window 8, hh 2, pinned [0], retrieval 2 frames, bf16); backbone replaced by synthetic "
            "q/k/v, points from a synthetic smooth depth surface")


# ------------------------------------------------------------------------------------ inputs
def synth_points(n_chunks, seed=0, sway=1.0):
    """Per chunk: points [chunk*tpf, 3] fp32 and mask [chunk*tpf] bool.  A hand-held pinhole camera
    hovers in front of a smooth depth surface that is fixed in the world (depth in [1, 10] m): it
    sways a few centimetres (sines of incommensurate periods plus millimetre jitter) and drifts
    slowly sideways, so the same 5 cm voxels are seen again and again, buffer rows fill up, pivots
    form, saturate and are re-merged, while new voxels keep appearing at the edge of the view.
    Patch centres of a 37 x 28 grid are unprojected onto the surface; the 5 special tokens of each
    frame carry zero points and are masked out (stream_session.py:249-255).  `sway` scales the
    camera motion (larger = more new voxels per frame)."""
    rs = np.random.RandomState(seed)
    c = CFG
    ph, pw = c["patch_h"], c["patch_w"]
    u = (np.arange(pw) + 0.5) / pw - 0.5
    v = (np.arange(ph) + 0.5) / ph - 0.5
    uu, vv = np.meshgrid(u, v)
    x, y = uu * 1.2, vv * 0.9
    freq = rs.rand(4, 2) * 3 + 0.5
    phase = rs.rand(4) * 2 * np.pi
    amp = rs.rand(4)
    out = []
    frame = 0
    two_pi = 2 * math.pi
    for _ in range(n_chunks):
        pts = np.zeros((c["chunk"] * c["tpf"], 3), np.float32)
        mask = np.zeros(c["chunk"] * c["tpf"], bool)
        for f in range(c["chunk"]):
            t = frame
            pos = np.array([0.08 * math.sin(two_pi * t / 97) + 0.0002 * t,
                            0.0125 * math.sin(two_pi * t / 53),
                            0.025 * math.sin(two_pi * t / 61)]) * sway + rs.randn(3) * 0.0005 * sway
            yaw = (0.01 * math.sin(two_pi * t / 131) + 0.00025 * rs.randn()) * sway
            cs, sn = math.cos(yaw), math.sin(yaw)
            depth = np.full_like(x, 5.0)
            for _it in range(3):      # fixed-point intersection of the pixel rays with the surface
                wx = cs * x * depth + sn * depth + pos[0]
                wy = y * depth + pos[1]
                surf = 5.5 + 4.5 * sum(a * np.sin(fr[0] * wx * 0.5 + fr[1] * wy * 0.5 + p_)
                                       for a, fr, p_ in zip(amp, freq, phase)) / amp.sum()
                depth = np.clip(surf, 1.0, 10.0) - pos[2]
            cam = np.stack([x * depth, y * depth, depth], -1).reshape(-1, 3)
            world = np.stack([cs * cam[:, 0] + sn * cam[:, 2], cam[:, 1], -sn * cam[:, 0] + cs * cam[:, 2]], 1) + pos
            lo = f * c["tpf"] + c["special"]
            pts[lo:lo + ph * pw] = world.astype(np.float32)
            mask[lo:lo + ph * pw] = rs.rand(ph * pw) < 0.95
            frame += 1
        out.append((pts, mask))
    return out


def retrieval_due(chunk_idx):
    """The reference's schedule (stream_session.py:478-489) for retrieval_size > 0."""
    c = CFG
    frame_idx = chunk_idx * c["chunk"]
    buffer_size = c["chunk"] + len(c["pinned"]) + c["window"] + c["hh"]
    if frame_idx <= max(buffer_size, 16):
        return False
    per_window = max(1, c["window"] // c["chunk"])
    return (frame_idx // c["chunk"] + 1) % per_window == 0


# ------------------------------------------------------------------------------------ clocks
class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons of one GPU every 50 ms while the timed region
    runs (one long-lived nvidia-smi process; read-only queries)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.proc = index, [], None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                parts = [x.strip() for x in line.strip().split(",")]
                if len(parts) >= 7:
                    self.rows.append(parts)
        except Exception:
            pass

    def stop(self):
        time.sleep(0.06)
        if self.proc is not None:
            self.proc.terminate()
        self.join(timeout=5)

        def num(x):
            try:
                return float(x)
            except ValueError:
                return None
        sm = [num(r[0]) for r in self.rows if num(r[0]) is not None]
        mx = [num(r[1]) for r in self.rows if num(r[1]) is not None]
        pw = [num(r[2]) for r in self.rows if num(r[2]) is not None]
        reasons = set()
        for r in self.rows:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(self.rows)}


# ------------------------------------------------------------------------------------ ours
class Stream:
    """One STAC stream on one GPU, driven like StreamSession.pipeline drives the manager."""

    def __init__(self, device, n_input_sets=3, seed=0, heads=None):
        import torch
        from stac_b200.stac import STACVoxelKV
        c = dict(CFG)
        if heads is not None:
            # head-sharded stream: this rank owns `heads` of the 16 heads and the same share of the
            # bounded voxel memory (2 M slots per layer for all heads together)
            c["max_buffer_slots"] = c["max_buffer_slots"] * heads // c["heads"]
            c["max_pivot_slots"] = c["max_pivot_slots"] * heads // c["heads"]
            c["heads"] = heads
        self.cfg = c
        self.torch, self.dev = torch, device
        buffer_size = c["chunk"] + len(c["pinned"]) + c["window"] + c["hh"]
        self.kv = STACVoxelKV(num_layers=c["layers"], num_heads=c["heads"], head_dim=c["head_dim"],
                              token_per_frame=c["tpf"], buffer_size=buffer_size, chunk_size=c["chunk"],
                              recent_size=c["window"], pinned_idx=c["pinned"], hh_size=c["hh"],
                              temperature=c["temperature"], device=device, dtype=torch.bfloat16,
                              voxel_size=c["voxel_size"], init_voxels=c["init_voxels"], voxel_buf_cap=c["buf_cap"],
                              voxel_piv_cap=c["piv_cap"], voxel_backend="cuda", sim_threshold=0.8,
                              replace_threshold=0.8, score_threshold=0.2, slab_growth=1024, slab_cap=10000,
                              seg_size=1, retrieval_size=c["retrieval"], allocator="segment", attn_backend="cuda",
                              max_buffer_slots=c["max_buffer_slots"], max_pivot_slots=c["max_pivot_slots"])
        self.kv.reset()
        Tq, H, D, L = c["chunk"] * c["tpf"], c["heads"], c["head_dim"], c["layers"]
        g = torch.Generator(device="cpu").manual_seed(seed)
        # host (pinned) master copies; device copies for the resident mode
        self.host = []
        for _ in range(n_input_sets):
            q = (torch.randn(L, 1, Tq, H, D, generator=g) / 8 * 4).to(torch.bfloat16).pin_memory()
            k = (torch.randn(L, 1, H, Tq, D, generator=g) / 8 * 4).to(torch.bfloat16).pin_memory()
            v = (torch.randn(L, 1, H, Tq, D, generator=g) / 8).to(torch.bfloat16).pin_memory()
            self.host.append((q, k, v))
        self.resident = [tuple(t.to(device) for t in s) for s in self.host]
        self.stage = [tuple(torch.empty_like(t, device=device) for t in self.host[0]) for _ in range(2)]
        n_tok = c["chunk"] * c["tpf"]
        self.stage_pts = [(torch.empty((n_tok, 3), dtype=torch.float32, device=device),
                           torch.empty(n_tok, dtype=torch.bool, device=device)) for _ in range(2)]
        self.pin_pts = [torch.empty((n_tok, 3), dtype=torch.float32).pin_memory() for _ in range(2)]
        self.pin_mask = [torch.empty(n_tok, dtype=torch.bool).pin_memory() for _ in range(2)]
        self.copy_stream = torch.cuda.Stream(device=device)
        self.ready = [None, None]
        self.done = [None, None]
        # results land in pinned memory; the host consumes the result of step i while step i + 1 runs
        self.out_host = [torch.empty((1, Tq, H, D), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        self.out_landed = [None, None]
        self.out_checksum = 0.0
        self.chunk_idx = 0
        self.share_counts = False
        self.head_counts = None
        self.attn_events = []
        self.prune_events = []
        self.query_counts = []       # device scalars: voxels queried by each retrieval of the timed steps
        self.h2d = self.d2h = 0

    def _prefetch(self, chunk_idx, pts, mask):
        """Host -> device copies of one step's q/k/v and points on the copy stream, into the
        staging set that step will read; waits until the compute that last read that set is done."""
        torch = self.torch
        slot = chunk_idx & 1
        s = chunk_idx % len(self.host)
        with torch.cuda.stream(self.copy_stream):
            if self.done[slot] is not None:
                self.copy_stream.wait_event(self.done[slot])
            self.pin_pts[slot].copy_(torch.from_numpy(pts))
            self.pin_mask[slot].copy_(torch.from_numpy(mask))
            self.stage_pts[slot][0].copy_(self.pin_pts[slot], non_blocking=True)
            self.stage_pts[slot][1].copy_(self.pin_mask[slot], non_blocking=True)
            # layer by layer, one event each: layer l of the step starts as soon as its own q/k/v have
            # landed, so even a step whose copies could not be issued ahead overlaps them with compute
            events = []
            for l in range(self.cfg["layers"]):
                for dst, src in zip(self.stage[slot], self.host[s]):
                    dst[l].copy_(src[l], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
                events.append(ev)
            self.ready[slot] = events

    def step(self, pts, mask, host_io=False, time_kernels=False, next_inputs=None):
        torch, kv, c = self.torch, self.kv, self.cfg
        L = c["layers"]
        s = self.chunk_idx % len(self.host)
        h2d = d2h = 0
        if host_io:
            # inputs of this step were staged by the copy stream (prefetched during the
            # previous step's compute); stage the next step's inputs into the other set now
            slot = self.chunk_idx & 1
            if self.ready[slot] is None:
                self._prefetch(self.chunk_idx, pts, mask)
            ready = self.ready[slot]
            q, k, v = self.stage[slot]
            pts_d, mask_d = self.stage_pts[slot]
            h2d = sum(t.numel() * 2 for t in self.host[s]) + pts.nbytes + mask.nbytes
            if next_inputs is not None:
                self._prefetch(self.chunk_idx + 1, *next_inputs)
        else:
            q, k, v = self.resident[s]
            pts_d, mask_d = pts, mask  # already device tensors
        out = None
        for l in range(L):
            if host_io:
                torch.cuda.current_stream().wait_event(ready[l])
            kv.append_kv(k[l], v[l], l)
            if time_kernels:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            out = kv.decode_sparse_attn(q[l], l)
            if time_kernels:
                e1.record()
                self.attn_events.append((e0, e1, q.shape[2], kv.get_offset()[l] + kv.get_retrieval_size()[l]))
        kv.append_positions(pts_d, mask_d)
        if retrieval_due(self.chunk_idx):
            for l in range(L):
                kv.retrieve_kv(l, return_buf=True)
            if time_kernels and kv._recent_voxel_ids is not None:
                self.query_counts.append(kv._recent_voxel_ids[1])
            if self.share_counts and kv._ret is not None:
                # head-sharded stream: every rank learns the valid pivot count of every head
                from stac_b200.sharding import gather_head_counts
                self.head_counts = gather_head_counts(kv._ret[2].sum(dim=1), L)
        if time_kernels:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        kv.prune_kv()
        if time_kernels:
            e1.record()
            self.prune_events.append((e0, e1))
        if host_io:
            slot = self.chunk_idx & 1
            self.out_host[slot].copy_(out, non_blocking=True)
            d2h += out.numel() * 2
            ev = torch.cuda.Event()
            ev.record()
            self.done[slot] = ev
            self.out_landed[slot] = ev
            self.ready[slot] = None
            # consume the previous step's result on the host (waits until its copy has landed);
            # the result of the last step is consumed by finish_host_io()
            prev = self.out_landed[1 - slot]
            if prev is not None:
                prev.synchronize()
                self.out_checksum += float(self.out_host[1 - slot][0, 0, 0, 0])
                self.out_landed[1 - slot] = None
        self.chunk_idx += 1
        self.h2d, self.d2h = h2d, d2h


def finish_host_io(stream):
    """Wait for and consume the results still in flight (end of a host-buffer phase)."""
    for slot in (0, 1):
        ev = stream.out_landed[slot]
        if ev is not None:
            ev.synchronize()
            stream.out_checksum += float(stream.out_host[slot][0, 0, 0, 0])
            stream.out_landed[slot] = None


def bench_config(world, shard_heads, K, W):
    """The `config` object of the JSON line; the same for both arms at the same N, K, W."""
    c = CFG
    return {"workload": WORKLOAD, "frames_per_step": c["chunk"], "streams": 1 if shard_heads else world,
            "frames_timed": c["chunk"] * K, "frames_before_timed_region": c["chunk"] * (c["prefill_chunks"] + W),
            "l2_policy": "inputs larger than L2 (hot cache 1.5 GB per stream, rotating q/k/v sets)",
            "prefill_chunks": c["prefill_chunks"],
            "masked_keys": "retrieved pivots beyond a head's valid count carry bias -inf; attention FLOPs count "
                           "all keys, `roofline.live_key_fraction` gives the share that is not masked",
            "parallelism": (f"1 stream, {c['heads']} heads sharded over {world} ranks (voxel memory sharded by head, "
                            "NCCL all-gather of per-head retrieval counts)") if shard_heads
            else f"{world} independent stream(s)"}


def max_over_ranks(ms, device=None):
    """Timed-region length of the job = the slowest rank's (device-timed) milliseconds."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(ms)
    t = torch.tensor([float(ms)], device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def job_throughput(frames_per_rank, ms, world):
    """Whole-job frames/s: every rank streams `frames_per_rank` frames in `ms` (max over ranks)."""
    return frames_per_rank * world / (ms / 1e3)


def exp2_bound(achieved_tf, clocks, dev):
    """Second limit of the attention pair at head_dim 64: one exponential per score in each of the
    two passes, 16 per clock per SM (measured with a stand-alone loop), i.e. (4+2r)*D = 384 flop
    per two exponentials.  Reported beside the tensor roofline; not the fraction that is judged."""
    import torch
    mhz = (clocks or {}).get("sm_mhz") or (clocks or {}).get("sm_max_mhz")
    if not mhz or not achieved_tf:
        return None
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
    cap = 16.0 * n_sm * mhz * 1e6 / 2.0 * 6 * CFG["head_dim"] / 1e12
    return {"tflops": round(cap, 1), "frac": round(achieved_tf / cap, 4), "at_sm_mhz": mhz,
            "rule": "2*H*M*N exponentials per call at 16 per clock per SM; a share of them runs on the FMA pipes"}


def attn_flops(M, N, r=1.0, heads=None):
    return (4.0 + 2.0 * r) * (heads or CFG["heads"]) * M * N * CFG["head_dim"]


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import __graft_entry__
    if rank == 0 and not os.path.exists(os.path.join(ROOT, "stac_b200", "libstac_b200.so")):
        __graft_entry__.build()
    if world > 1:
        dist.barrier()
    c = CFG
    K, W = args.steps, max(args.warmup, 3)
    n_chunks = c["prefill_chunks"] + 2 * (W + K)
    shard_heads = args.shard == "heads" and world > 1
    if shard_heads:
        from stac_b200.sharding import head_slice
        hs = head_slice(rank, world, c["heads"])
        local_heads = hs.stop - hs.start
        points = synth_points(n_chunks, seed=0)       # one stream: every rank sees the same points
        stream = Stream(dev, seed=rank, heads=local_heads)
        stream.share_counts = True
    else:
        local_heads = c["heads"]
        points = synth_points(n_chunks, seed=rank)
        stream = Stream(dev, seed=rank)
    pts_dev = [(torch.from_numpy(p).to(dev), torch.from_numpy(m).to(dev)) for p, m in points]
    it = iter(range(n_chunks))

    def run_phase(n, host_io, timed):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k_step in range(n):
            i = next(it)
            if host_io:
                # prefetch only inside the phase: every timed step's copies start in the timed region
                nxt = points[i + 1] if (k_step + 1 < n and i + 1 < len(points)) else None
                stream.step(points[i][0], points[i][1], host_io=True, next_inputs=nxt)
            else:
                stream.step(pts_dev[i][0], pts_dev[i][1], time_kernels=timed)
        e1.record()
        if host_io:
            finish_host_io(stream)
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1), dev)

    run_phase(c["prefill_chunks"], False, False)   # fill the hot cache, start eviction + retrieval
    run_phase(W, False, False)                     # warm-up
    from stac_b200 import _lib as stac_lib
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.25)
    launches0 = stac_lib.kernel_launches()
    torch.cuda.nvtx.range_push("timed_steps")      # lets a profiler pick exactly the timed steps
    stream.kv.stage_trace = []                     # per-stage CUDA events of the timed steps
    ms_dev = run_phase(K, False, True)             # timed, device-resident inputs
    torch.cuda.nvtx.range_pop()
    launches = stac_lib.kernel_launches() - launches0
    clocks = sampler.stop()
    trace, stream.kv.stage_trace = stream.kv.stage_trace, None
    run_phase(min(W, 3), True, False)              # warm the host path
    ms_e2e = run_phase(K, True, False)             # timed, host buffers
    stream.kv.check_status()
    copy_gbs = h2d_copy_ceiling(stream, dev)       # the same copies with no compute behind them

    n_streams = 1 if shard_heads else world
    value = job_throughput(c["chunk"] * K, ms_dev, n_streams)
    e2e = job_throughput(c["chunk"] * K, ms_e2e, n_streams)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak_tf = peaks.get("bf16_tflops_sustained", 1400.0)
    peak_hbm = peaks.get("hbm_gbs", 6650.0)
    peak_src = "measured (MEASURED_PEAKS.json)" if peaks else "fallback (1.4 PFLOP/s sustained, 6.65 TB/s)"
    # ---- roofline of the dominant kernel pair (attention forward + column sums), per call
    att_ms, att_fl = [], []
    for e0, e1, M, N in stream.attn_events:
        att_ms.append(e0.elapsed_time(e1))
        att_fl.append(attn_flops(M, N, heads=local_heads))
    achieved = sum(att_fl) / (sum(att_ms) / 1e3) / 1e12 if att_ms else None
    # ---- the memory-bound stages, timed inside the same steps
    prune_ms = [e0.elapsed_time(e1) for e0, e1 in stream.prune_events]
    stage_ms = {}
    for name, e0, e1 in trace:
        stage_ms.setdefault(name, []).append(e0.elapsed_time(e1))
    LH, D, eb = c["layers"] * local_heads, c["head_dim"], 2
    T_d = c["chunk"] * c["tpf"]                     # tokens evicted per (layer, head) per steady-state step
    R = c["retrieval"] * c["tpf"]
    T_keep = (len(c["pinned"]) + c["window"] + c["hh"]) * c["tpf"]
    q_counts = [int(t.item()) for t in stream.query_counts]
    Q = float(np.mean(q_counts)) if q_counts else 0.0

    def mem_roof(stage, nbytes, formula):
        if stage not in stage_ms:
            return None
        ms = float(np.mean(stage_ms[stage]))
        gbs = nbytes / ms / 1e6
        return {"kernel": stage, "bytes": int(nbytes), "bytes_formula": formula, "ms": round(ms, 4),
                "calls": len(stage_ms[stage]), "gbs": round(gbs, 1), "peak": peak_hbm,
                "frac": round(gbs / peak_hbm, 4), "unit": "GB/s"}
    roof_mem = {
        "merge": mem_roof("merge", LH * T_d * (4 * D * eb + 12), "E*(4*D*e+12), E = L*H*T_d evicted tokens"),
        "retrieve": mem_roof("retrieve", LH * R * (4 * D * eb + 5) + LH * Q * c["piv_cap"] * 12,
                             "L*H*R*(4*D*e+5) + L*H*Q*P*12, Q = queried voxels"),
        "compact": mem_roof("compact", LH * T_keep * (4 * D * eb + 24), "L*H*T_keep*(4*D*e+24)"),
        "h2o_select": mem_roof("h2o_select", LH * (T_keep + T_d) * 8, "L*H*T*(4 read + 4 written)"),
    }
    info = stream.kv.get_merger_info()
    ret_valid = None
    if stream.kv._ret is not None:
        per_head = stream.kv._ret[2].sum(dim=1).float()
        ret_valid = {"mean_per_head": round(float(per_head.mean()), 1), "min_per_head": int(per_head.min()),
                     "of": R, "fraction": round(float(per_head.mean()) / R, 4)}
    live_frac = None
    if ret_valid is not None and att_ms:
        N_full = T_keep + T_d + R
        live_frac = round((T_keep + T_d + ret_valid["mean_per_head"]) / N_full, 4)
    h2d_gbs = stream.h2d / (ms_e2e / K) / 1e6 if stream.h2d else None
    line = {
        "metric": METRIC, "value": round(value, 3), "unit": "frames/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(ms_dev / K, 4), "higher_is_better": True,
        "scaling": "strong" if shard_heads else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": bench_config(world, shard_heads, K, W),
        "e2e": {"value": round(e2e, 3), "unit": "frames/s", "h2d_bytes_per_step": stream.h2d,
                "d2h_bytes_per_step": stream.d2h, "ms_per_step": round(ms_e2e / K, 4),
                "h2d_gbs_per_rank": round(h2d_gbs, 1) if h2d_gbs else None,
                "h2d_copy_only_gbs_per_rank": round(copy_gbs, 1) if copy_gbs else None},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "attn_fwd_fast_kernel + attn_colsum_kernel (one call per layer)",
                     "achieved": round(achieved, 2) if achieved else None, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": round(achieved / peak_tf, 4) if achieved else None, "peak_source": peak_src,
                     "flops_formula": "(4+2r)*H*M*N*D, r=1, N = all keys", "live_key_fraction": live_frac,
                     "avg_ms_per_call": round(float(np.mean(att_ms)), 4),
                     # dram__bytes_read.sum + dram__bytes_write.sum of the two kernels of one call at
                     # this shape (M=4164, N=17697), one ncu capture per kernel
                     "traffic": ATTN_TRAFFIC_BYTES_PER_CALL,
                     "traffic_unit": "bytes per call (fwd 84.7 + 8.8 MB, colsum 45.4 MB; algorithmic 135 MB)",
                     "exp2_unit_bound": exp2_bound(achieved, clocks, dev)},
        "roofline_memory": roof_mem,
        "stages_ms_per_step": dict({"attention_24_layers": round(sum(att_ms) / K, 3),
                                    "prune_total": round(sum(prune_ms) / K, 3)},
                                   **{k_: round(sum(v_) / K, 4) for k_, v_ in stage_ms.items()}),
        "pool": {"voxels": info["used_voxels"], "pivots": info["pivot_pool_used"],
                 "buffered": info["buffer_pool_used"], "buffer_slots_max": stream.cfg["max_buffer_slots"],
                 "pivot_slots_max": stream.cfg["max_pivot_slots"], "dropped_tokens": info["dropped_tokens"],
                 "tokens_evicted": info["token_count"], "retrieved_valid_pivots": ret_valid,
                 "queried_voxels_mean": round(Q, 1)},
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(sample_seconds=15.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def h2d_copy_ceiling(stream, dev, reps=3):
    """GB/s of the e2e leg's host -> device copies (one step's q/k/v, layer by layer, from the same
    pinned buffers into the same staging set) with no compute behind them: what the host side of
    this box can deliver to this rank while the other ranks do the same."""
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()
    nbytes = sum(t.numel() * 2 for t in stream.host[0])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream.copy_stream):
        e0.record()
        for r in range(reps):
            for l in range(stream.cfg["layers"]):
                for dst, src in zip(stream.stage[r & 1], stream.host[r % len(stream.host)]):
                    dst[l].copy_(src[l], non_blocking=True)
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    return nbytes * reps / ms / 1e6 if ms > 0 else None


# ------------------------------------------------------------------------------------ microbenchmarks
def run_microbench_attn(args):
    """Column-sum attention microbenchmark: bf16 q [1041,16,64] against Lk keys; prints one JSON line per run with
    TFLOP/s counted as (4+2r)*H*M*N*D.  Used for kernel profiling; not the headline line."""
    import torch
    from stac_b200 import ops
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    H, D, M, Lk = CFG["heads"], CFG["head_dim"], args.m, args.lk
    n_ret = min(args.pivots, Lk)
    T_hot = Lk - n_ret
    q = (torch.randn(M, H, D, device=dev) / 8).to(torch.bfloat16)
    sets = []
    for _ in range(3):   # rotate inputs so that K/V do not stay in L2 between iterations
        k = (torch.randn(H, Lk, D, device=dev) / 8).to(torch.bfloat16)
        v = (torch.randn(H, Lk, D, device=dev) / 8).to(torch.bfloat16)
        sets.append((k, v))
    bias = torch.log(torch.randint(1, 9, (H, max(n_ret, 1)), device=dev).float())
    bias[torch.rand(H, max(n_ret, 1), device=dev) < 0.25] = float("-inf")
    st = ops.DeviceStatus(dev)

    def call(i):
        k, v = sets[i % 3]
        if n_ret:
            return ops.attn_colsum(q, k, v, T_hot, k[:, T_hot:], v[:, T_hot:], bias, n_ret, status=st)
        return ops.attn_colsum(q, k, v, Lk, status=st)

    for i in range(max(args.warmup, 3)):
        call(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        call(i)
    e1.record()
    host_us = (time.perf_counter() - t0) / args.steps * 1e6
    torch.cuda.synchronize()
    st.raise_if_set("attention microbench")
    eager_ms = e0.elapsed_time(e1) / args.steps
    # The same calls replayed from a CUDA graph (24 calls, one per layer of a chunk): at the
    # short shapes a call's kernels take less time than the Python and ctypes work of issuing
    # them, so the eager loop measures the host.  `value` is the graph figure.
    side = torch.cuda.Stream()
    n_graph = 24
    with torch.cuda.stream(side):
        for i in range(3):
            call(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            keep = [call(i) for i in range(n_graph)]
        reps = max(1, (args.steps + n_graph - 1) // n_graph)
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        e0.record(side)
        for _ in range(reps):
            graph.replay()
        e1.record(side)
        torch.cuda.synchronize()
    st.raise_if_set("attention microbench (graph)")
    ms = e0.elapsed_time(e1) / (reps * n_graph)
    del keep
    tf = attn_flops(M, Lk) / (ms / 1e3) / 1e12
    print(json.dumps({"metric": "attn_colsum_tflops", "value": round(tf, 2), "unit": "TFLOP/s",
                      "ms_per_call": round(ms, 4), "timing": f"CUDA graph of {n_graph} calls, {reps} replays",
                      "eager_ms_per_call": round(eager_ms, 4), "eager_tflops": round(attn_flops(M, Lk) / eager_ms / 1e9, 2),
                      "host_us_per_call": round(host_us, 1), "steps": args.steps,
                      "config": {"workload": f"config2 attention microbench M={M} Lk={Lk} pivots={n_ret} H=16 D=64 bf16"}}))


def run_microbench_pointmap(args):
    """Point maps of one chunk (4 frames, 518 x 392) -> patch points + mask -> voxel ids: the
    fused kernel against the reference's torch sequence (permute, two interpolates, reshape, cat)
    on the same device, both followed by the same voxel upsert."""
    import torch
    from stac_b200 import _lib
    from stac_b200.stac.pointmap import pointmap_to_positions
    dev = torch.device("cuda:0")
    S, H, W, patch, special = CFG["chunk"], 392, 518, 14, 5
    g = torch.Generator(device="cpu").manual_seed(0)
    wp = (torch.rand(1, S, H, W, 3, generator=g) * 8 - 4).to(dev)
    cf = (torch.rand(1, S, H, W, generator=g) * 2).to(dev)

    def torch_path():
        p = wp.permute(0, 1, 4, 2, 3).view(-1, 3, H, W)
        c = cf.unsqueeze(-1).permute(0, 1, 4, 2, 3).view(-1, 1, H, W)
        ds = (H // patch, W // patch)
        p = torch.nn.functional.interpolate(p, size=ds, mode="bilinear", align_corners=False)
        c = torch.nn.functional.interpolate(c, size=ds, mode="bilinear", align_corners=False)
        p = torch.cat((p.new_zeros((S, special, 3)), p.permute(0, 2, 3, 1).reshape(S, -1, 3)), dim=1)
        m = c.permute(0, 2, 3, 1).reshape(S, -1) > 1.0
        return p, torch.cat((m.new_zeros((S, special)), m), dim=1)

    def ours():
        return pointmap_to_positions(wp, cf, patch, 1.0, special)

    res = {}
    for name, fn in (("torch_sequence", torch_path), ("fused_kernel", ours)):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        res[name] = e0.elapsed_time(e1) / args.steps * 1e3
    a, b = torch_path(), ours()
    same = bool(torch.equal(a[1], b[1])) and float((a[0] - b[0]).abs().max()) < 1e-5
    n_tok = S * (special + (H // patch) * (W // patch))
    print(json.dumps({"metric": "pointmap_to_positions_us", "value": round(res["fused_kernel"], 2), "unit": "us",
                      "torch_sequence_us": round(res["torch_sequence"], 2), "tokens": n_tok,
                      "algorithmic_bytes": n_tok * (4 * 16 + 13), "agrees_with_torch_sequence": same,
                      "kernels": _lib.kernel_launches(), "steps": args.steps,
                      "config": {"workload": f"point maps {S} x {H} x {W} -> {n_tok} patch points (latency-bound)"}}))


def run_config3(args):
    """Voxel pool stress as the configuration states it: 24 layers x 16 heads x 64 bf16 (384 pool
    heads), buffer and pivot pools bounded at 1 M slots each, 8 frames (8328 tokens per head)
    evicted per step with points from the synthetic depth surface, `--steps` steps (512) of merge
    each followed by retrieval of the top 2048 pivots per head around that step's voxels.
    Prints one JSON line: median and p95 milliseconds and GB/s (algorithmic bytes) of both calls,
    pivots formed, tokens dropped by the bounded pool."""
    import torch
    from stac_b200 import ops
    from stac_b200.stac.merger import VoxelKVMerger
    from stac_b200.stac.voxel import BinaryVoxel
    dev = torch.device("cuda", 0)
    c = CFG
    LH, D, Td, R = c["layers"] * c["heads"], c["head_dim"], args.m, 2048
    slots = args.pool_slots
    st = ops.DeviceStatus(dev)
    vm = BinaryVoxel(c["voxel_size"], dev, status=st)
    mg = VoxelKVMerger(LH, D, init_voxels=c["init_voxels"], pivot_cap=4, budget_cap=8, sim_thresh=0.8,
                       replace_thresh=0.8, score_thresh=0.2, dtype=torch.bfloat16, device=dev, status=st,
                       max_buffer_slots=slots, max_pivot_slots=slots)
    torch.manual_seed(0)
    n_steps = args.warmup + args.steps
    per_chunk = c["chunk"] * c["tpf"]
    chunks = synth_points((n_steps * Td + per_chunk - 1) // per_chunk + 1, seed=0)
    allpts = np.concatenate([p for p, _ in chunks])
    allmask = np.concatenate([m for _, m in chunks])
    sets = [((torch.randn(LH, Td, D, device=dev)).to(torch.bfloat16), (torch.randn(LH, Td, D, device=dev)).to(torch.bfloat16),
             torch.rand(LH, Td, device=dev)) for _ in range(3)]      # rotate: 3 x 0.8 GB > L2
    times_m, times_r, q_sizes = [], [], []
    for step in range(n_steps):
        pts = torch.from_numpy(allpts[step * Td:(step + 1) * Td]).to(dev)
        msk = torch.from_numpy(allmask[step * Td:(step + 1) * Td]).to(dev)
        ids = vm.upsert_points(pts, msk)
        VX = ids.view(1, -1).expand(LH, -1).contiguous()
        K, V, S = sets[step % 3]
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        e[0].record()
        mg.insert_evicted(K, V, S, VX, None, Td, vm.voxel_num_bound(), voxel_count_dev=vm._n_dev)
        e[1].record()
        q_ids, q_cnt = vm.neighbor_ids(ids, 2)
        e[2].record()
        mg.retrieve_device(q_ids, q_cnt, R)
        e[3].record()
        torch.cuda.synchronize()
        if step >= args.warmup:
            times_m.append(e[0].elapsed_time(e[1]))
            times_r.append(e[2].elapsed_time(e[3]))
            q_sizes.append(int(q_cnt.item()))
    st.raise_if_set("voxel pool stress")
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = peaks.get("hbm_gbs", 6650.0)
    E = LH * Td
    bytes_m = E * (4 * D * 2 + 12)
    bytes_r = LH * R * (4 * D * 2 + 5) + LH * float(np.mean(q_sizes)) * 4 * 12
    tm, tr = np.array(times_m), np.array(times_r)

    def stats(t, nbytes):
        med, p95 = float(np.median(t)), float(np.percentile(t, 95))
        return {"median_ms": round(med, 4), "p95_ms": round(p95, 4), "max_ms": round(float(t.max()), 3),
                "gbs_at_median": round(nbytes / med / 1e6, 1), "gbs_at_p95": round(nbytes / p95 / 1e6, 1),
                "frac_of_peak_at_median": round(nbytes / med / 1e6 / peak, 4), "algorithmic_bytes": int(nbytes)}
    info = mg.info()
    print(json.dumps({"metric": "voxel_pool_stress_merge_hbm_gbs", "value": stats(tm, bytes_m)["gbs_at_median"],
                      "unit": "GB/s", "steps": args.steps, "warmup": args.warmup, "peak_gbs": peak,
                      "merge": stats(tm, bytes_m), "retrieve": stats(tr, bytes_r),
                      "queried_voxels_mean": round(float(np.mean(q_sizes)), 1),
                      "pool": {"slots_per_pool": slots, "voxels": info["used_voxels"], "pivots": info["pivot_pool_used"],
                               "buffered": info["buffer_pool_used"], "tokens_evicted": info["token_count"],
                               "dropped_tokens": info["dropped_tokens"]},
                      "config": {"workload": f"config3 voxel pool stress: 384 pool heads x {Td} evicted tokens/step, bf16, "
                                             f"pools bounded at {slots} slots, synthetic depth surface, retrieve top-{R} "
                                             "per head after every merge"}}))


# ------------------------------------------------------------------------------------ CPU arm
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
CPU_SAMPLE = (2, 4)      # (layers, heads) of the stream that the CPU arms run: 8 of the 384 (layer, head) rows


def _reference_available():
    return os.path.isfile(os.path.join(REF_DIR, "stac", "stac_voxel.py"))


class ReferenceCpuStream:
    """The reference's OWN manager (stac/stac_voxel.py STACVoxelKV with voxel_backend="python",
    allocator="segment", seg_size=1, device="cpu", fp32: its CPU torch path) driven through one
    chunk at a time on a subset of (layers, heads).  The reference has no CPU attention (its
    decode_sparse_attn asserts CUDA, stac/stac_voxel.py:217), so the attention is the fp32 torch
    computation of its own self-check (stac/flash_attn_triton.py:1018-1036) and the column sums
    are handed to its _update_scores exactly as decode_sparse_attn does (stac/stac_voxel.py:252-265)."""

    kind = "reference"

    def __init__(self, n_layers, n_heads, seed=0):
        import logging
        import torch
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        logging.disable(logging.INFO)
        from stac.stac_voxel import STACVoxelKV
        c = CFG
        self.torch, self.L, self.H = torch, n_layers, n_heads
        torch.set_num_threads(os.cpu_count() or 1)
        self.threads = torch.get_num_threads()
        buffer_size = c["chunk"] + len(c["pinned"]) + c["window"] + c["hh"]
        self.kv = STACVoxelKV(num_layers=n_layers, num_heads=n_heads, head_dim=c["head_dim"],
                              token_per_frame=c["tpf"], buffer_size=buffer_size, chunk_size=c["chunk"],
                              recent_size=c["window"], pinned_idx=list(c["pinned"]), hh_size=c["hh"],
                              temperature=c["temperature"], device=torch.device("cpu"), dtype=torch.float32,
                              voxel_size=c["voxel_size"], init_voxels=c["init_voxels"], voxel_buf_cap=c["buf_cap"],
                              voxel_piv_cap=c["piv_cap"], voxel_backend="python", sim_threshold=0.8,
                              replace_threshold=0.8, score_threshold=0.2, slab_growth=1024, slab_cap=10000,
                              seg_size=1, retrieval_size=c["retrieval"], allocator="segment", attn_backend="cuda")
        self.kv.reset()
        self.points = synth_points(64, seed=seed)
        self.gen = torch.Generator().manual_seed(seed)
        self.chunk = 0

    def step(self):
        torch, kv, c = self.torch, self.kv, CFG
        Tq, D, H = c["chunk"] * c["tpf"], c["head_dim"], self.H
        pts, mask = self.points[self.chunk % len(self.points)]
        t0 = time.perf_counter()
        with torch.no_grad():
            for l in range(self.L):
                q = torch.randn(H, Tq, D, generator=self.gen) / 2
                k = torch.randn(1, H, Tq, D, generator=self.gen) / 2
                v = torch.randn(1, H, Tq, D, generator=self.gen) / 8
                kv.append_kv(k, v, l)
                T = kv._offset_hot[l]
                K_all, V_all = kv.key_cache_hot[l][:, :T], kv.value_cache_hot[l][:, :T]
                T_ret = kv._offset_retrieval[l]
                scores = None
                if T_ret > 0:
                    K_all = torch.cat([K_all, kv.key_cache_retrieval[l][:, :T_ret]], 1)
                    V_all = torch.cat([V_all, kv.value_cache_retrieval[l][:, :T_ret]], 1)
                scores = torch.matmul(q, K_all.transpose(1, 2)) * (D ** -0.5)
                if T_ret > 0:
                    scores[:, :, T:] += kv._bias_retrieval[l][:, None, :T_ret]
                attn = torch.softmax(scores, dim=-1)
                colsum = attn.sum(dim=1)                    # [H, T + T_ret]
                _ = torch.matmul(attn, V_all)
                kv._last_query_offset[l] = Tq
                kv._update_scores(colsum[None, :, None, :T], l)
                del scores, attn
            kv.append_positions(torch.from_numpy(pts), torch.from_numpy(mask))
            if retrieval_due(self.chunk):
                for l in range(self.L):
                    kv.retrieve_kv(l, return_buf=True)
            kv.prune_kv()
        self.chunk += 1
        return time.perf_counter() - t0


class PortCpuStream:
    """Same sample through the numpy restatement of that path (oracle/), used when the staged
    reference sources (oracle/_ref) are absent."""

    kind = "port"

    def __init__(self, n_layers, n_heads, seed=0):
        self.n_layers, self.n_heads, self.state, self.seed = n_layers, n_heads, None, seed
        self.threads = os.cpu_count() or 1

    def step(self):
        dt, self.state = cpu_step_sample(self.n_layers, self.n_heads, self.state, seed=self.seed)
        return dt


def cpu_stream():
    n_layers, n_heads = CPU_SAMPLE
    return ReferenceCpuStream(n_layers, n_heads) if _reference_available() else PortCpuStream(n_layers, n_heads)


def cpu_step_sample(n_layers, n_heads, state=None, seed=0):
    """One chunk of the same workload through the CPU oracle on a subset of (layers, heads);
    returns seconds and the state for the next chunk."""
    from oracle.attention import attn_colsum
    from oracle.manager import StacManager
    c = CFG
    buffer_size = c["chunk"] + len(c["pinned"]) + c["window"] + c["hh"]
    if state is None:
        mg = StacManager(n_layers, n_heads, c["head_dim"], c["tpf"], buffer_size, chunk_size=c["chunk"],
                         recent_size=c["window"], pinned_idx=tuple(c["pinned"]), hh_size=c["hh"],
                         temperature=c["temperature"], voxel_size=c["voxel_size"], init_voxels=c["init_voxels"],
                         retrieval_size=c["retrieval"], dtype="bf16")
        state = {"mg": mg, "chunk": 0, "points": synth_points(64, seed=seed), "rs": np.random.RandomState(seed)}
    mg, rs = state["mg"], state["rs"]
    Tq, D = c["chunk"] * c["tpf"], c["head_dim"]
    pts, mask = state["points"][state["chunk"] % 64]
    t0 = time.perf_counter()
    for l in range(n_layers):
        q = (rs.randn(Tq, n_heads, D) / 2).astype(np.float32)
        k = (rs.randn(n_heads, Tq, D) / 2).astype(np.float32)
        v = (rs.randn(n_heads, Tq, D) / 8).astype(np.float32)
        mg.append_kv(k, v, l)
        T = mg.off[l]
        k_all = mg.K[l, :, :T].transpose(1, 0, 2)
        v_all = mg.V[l, :, :T].transpose(1, 0, 2)
        bias = None
        if mg.ret is not None:
            Kr, Vr, Br = mg.ret[0], mg.ret[1], mg.ret[2]
            sl = slice(l * n_heads, (l + 1) * n_heads)
            k_all = np.concatenate([k_all, Kr[sl].transpose(1, 0, 2)], 0)
            v_all = np.concatenate([v_all, Vr[sl].transpose(1, 0, 2)], 0)
            bias = np.concatenate([np.zeros((n_heads, T), np.float32), Br[sl]], 1)
        _, _, cs = attn_colsum(q, k_all, v_all, bias)
        mg.update_scores(cs[:, :T], l, Tq)
    mg.append_positions(pts, mask)
    if retrieval_due(state["chunk"]):
        mg.retrieve(return_buf=True)
    mg.prune()
    dt = time.perf_counter() - t0
    state["chunk"] += 1
    return dt, state


def _cpu_record(st, seconds, n_steps):
    """Fields common to `cpu_baseline` and the reference arm: what was measured and how it is scaled."""
    n_layers, n_heads = CPU_SAMPLE
    rows, all_rows = n_layers * n_heads, CFG["layers"] * CFG["heads"]
    scale = all_rows / rows
    fps = CFG["chunk"] * n_steps / (seconds * scale)
    what = ("the reference's own manager (stac/stac_voxel.py, voxel_backend=python, allocator=segment, fp32, CPU) "
            "with the fp32 torch attention of its self-check" if st.kind == "reference"
            else "numpy restatement of the reference's Python path (oracle/); oracle/_ref was not staged")
    return {"value": round(fps, 5), "unit": "frames/s", "cores": st.threads, "host_cpus": os.cpu_count(),
            "kind": st.kind, "sample_rows": rows, "all_rows": all_rows, "scale_factor": scale,
            "sample_seconds_measured": round(seconds, 3), "sample_steps": n_steps,
            "sample": f"{n_steps} steady-state chunks of {n_layers} layer x {n_heads} heads ({rows} of the {all_rows} "
                      f"(layer, head) rows, which are independent); measured {seconds:.2f} s, scaled x{scale:.0f} "
                      f"to the full stream; {what}; torch/BLAS threads = {st.threads}"}


def cpu_baseline(sample_seconds=15.0):
    """The reference's CPU path on this host on a bounded sample of the same stream (see
    ReferenceCpuStream); throughput is scaled by the sampled fraction of (layer, head) rows."""
    st = cpu_stream()
    for _ in range(5):            # reach the pruning regime (untimed)
        st.step()
    t, n = 0.0, 0
    while t < sample_seconds and n < 8:
        t += st.step()
        n += 1
    return _cpu_record(st, t, n)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    K, W = args.steps, max(args.warmup, 3)
    st = cpu_stream()
    for _ in range(4 + min(W, 3)):
        st.step()
    t = 0.0
    for _ in range(K):
        t += st.step()
    rec = _cpu_record(st, t, K)
    shard_heads = args.shard == "heads" and world > 1
    line = {"impl": "reference", "metric": METRIC, "value": rec["value"], "unit": "frames/s",
            "n_gpus": world, "steps": K, "warmup": W,
            # one step of the FULL workload at this rate (the sampled rows' seconds x scale_factor)
            "ms_per_step": round(t / K * 1e3 * rec["scale_factor"], 2),
            "ms_per_step_measured_on_sample": round(t / K * 1e3, 2),
            "higher_is_better": True, "scaling": "strong" if shard_heads else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": bench_config(world, shard_heads, K, W),
            "cpu_baseline": rec,
            "e2e": {"value": rec["value"], "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard", default="streams", choices=["streams", "heads"],
                    help="N > 1: one independent stream per GPU (default, weak scaling) or ONE stream whose heads "
                         "and voxel memory are sharded over the GPUs (strong scaling)")
    ap.add_argument("--microbench", default=None, choices=["attn", "merge", "pointmap"],
                    help="kernel microbenchmarks used for profiling (not the headline line); `merge` is the "
                         "voxel pool stress configuration (512 steps unless --steps is given)")
    ap.add_argument("--pool-slots", type=int, default=1_000_000, help="pool stress: slots of each bounded pool")
    ap.add_argument("--lk", type=int, default=10376, help="attention microbench: number of keys")
    ap.add_argument("--m", type=int, default=None, help="microbench: query rows (attn) / evicted tokens per head (merge)")
    ap.add_argument("--pivots", type=int, default=0, help="attention microbench: keys carrying a bias")
    a = ap.parse_args()
    if a.steps is None:
        a.steps = 512 if a.microbench == "merge" else 8
    if a.microbench == "attn":
        a.m = a.m or 1041
        run_microbench_attn(a)
    elif a.microbench == "merge":
        a.m = a.m or 8328
        run_config3(a)
    elif a.microbench == "pointmap":
        run_microbench_pointmap(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
