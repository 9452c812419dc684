"""CPU-side checks: the C ABI library loads and exports every declared symbol, the product
refuses to run without a GPU (no CPU fallback), bench helpers, and the multi-rank timing logic
on two gloo ranks."""

import os
import re
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "stac_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(stac_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__
    __graft_entry__.build()
    from stac_b200 import _lib
    import ctypes
    names = _declared_functions()
    assert len(names) >= 15
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/stac_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)
    lib = _lib.lib()
    assert lib.stac_abi_version() == 2
    assert lib.stac_status_string(1) == b"bad argument"
    # row log-sum-exps (+ 512 words of flags and counters, rounded up to 256 bytes) + two partial forward
    # results and two partial column-sum groups (3 x 128 keys) per CTA
    lse_bytes = ((1041 * 16 + 512) * 4 + 255) // 256 * 256
    assert lib.stac_attn_workspace_bytes(1041, 16) == lse_bytes + 2 * 160 * (128 * 64 + 2 * 128 + 3 * 128) * 4
    assert lib.stac_merge_scratch_bytes(4, 100, 1000) > 0
    assert lib.stac_voxel_scratch_bytes(10) == (10 + 16) * 8 + 16   # keys, key list padded to 16, counter


def test_struct_layout_matches_header():
    import ctypes
    from stac_b200 import _lib
    # 10 4-byte fields, 6 pointers + int (+pad), 7 pointers + int (+pad), 10 pointers, int (+pad), 2 pointers
    assert ctypes.sizeof(_lib.StacPool) == 40 + 6 * 8 + 8 + 7 * 8 + 8 + 10 * 8 + 8 + 8 + 8
    assert ctypes.sizeof(_lib.StacEvicted) == 8 * 8 + 8


def test_product_has_no_cpu_path():
    import torch
    from stac_b200 import _lib
    from stac_b200.stac import STACVoxelKV
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(_lib.StacError):
        STACVoxelKV(num_layers=1, num_heads=2, head_dim=64, token_per_frame=8, buffer_size=4,
                    device=torch.device("cpu"), dtype=torch.bfloat16)
    import stac_b200.stac.stac_voxel as sv
    src = open(sv.__file__).read() + open(os.path.join(ROOT, "stac_b200", "ops.py")).read()
    assert "oracle" not in src


def test_manager_rejects_unsupported_config():
    import torch
    from stac_b200.stac.merger import VoxelKVMerger
    with pytest.raises(ValueError):
        VoxelKVMerger(4, 64, budget_cap=32, dtype=torch.bfloat16, device="cpu")
    with pytest.raises(ValueError):
        VoxelKVMerger(4, 128, budget_cap=8, dtype=torch.bfloat16, device="cpu")


def test_bench_helpers():
    sys.path.insert(0, ROOT)
    import bench
    pts = bench.synth_points(3, seed=1)
    pts2 = bench.synth_points(3, seed=1)
    tpf, ck = bench.CFG["tpf"], bench.CFG["chunk"]
    assert pts[0][0].shape == (ck * tpf, 3) and pts[0][1].shape == (ck * tpf,)
    assert all(np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]) for a, b in zip(pts, pts2))
    assert not pts[0][1][:5].any() and not pts[0][1][tpf:tpf + 5].any()     # special tokens masked
    z = pts[1][0][pts[1][1]]
    assert np.isfinite(z).all()
    due = [i for i in range(12) if bench.retrieval_due(i)]
    assert due == [5, 7, 9, 11]
    assert bench.attn_flops(1041, 10376) == 6 * 16 * 1041 * 10376 * 64
    assert bench.job_throughput(32, 1000.0, 8) == 256.0


def test_cpu_arms_of_the_bench_step(monkeypatch):
    """The two CPU legs of bench.py (`cpu_baseline`, `--impl reference`): one chunk of one layer and
    one head through the numpy port and, where its sources are staged, through the reference's
    own manager; the record says what was measured and how it is scaled."""
    sys.path.insert(0, ROOT)
    import bench
    monkeypatch.setattr(bench, "CPU_SAMPLE", (1, 1))
    arms = [bench.PortCpuStream(1, 1)]
    if bench._reference_available():
        arms.append(bench.ReferenceCpuStream(1, 1))
    for st in arms:
        dt = st.step() + st.step()
        assert dt > 0.0
        rec = bench._cpu_record(st, dt, 2)
        assert rec["kind"] == st.kind and rec["scale_factor"] == 384.0 and rec["sample_rows"] == 1
        assert rec["value"] == round(bench.CFG["chunk"] * 2 / (dt * 384.0), 5)
        assert rec["cores"] >= 1 and "scaled x384" in rec["sample"]


def _rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    import bench
    dist.barrier()
    ms = bench.max_over_ranks(100.0 + 50.0 * rank)
    q.put((rank, ms, bench.job_throughput(16, ms, world)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_timing_is_max_over_ranks():
    """world_size 2 on gloo: each rank streams independently; the job time is the slower rank's."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [150.0, 150.0]
    assert all(abs(r[2] - 32 / 0.15) < 1e-9 for r in res)


def _shard_rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from stac_b200.sharding import gather_head_counts, head_slice
    L, H = 3, 8
    full = torch.arange(L * H, dtype=torch.int32).reshape(L, H) * 7 % 11
    sl = head_slice(rank, world, H)
    got = gather_head_counts(full[:, sl].reshape(-1), L)
    q.put((rank, got.tolist(), full.tolist(), [sl.start, sl.stop]))
    dist.barrier()
    dist.destroy_process_group()


def test_head_sharding_counts_two_ranks():
    """Head-sharded stream: every rank ends with the per-head retrieval counts of all heads."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000
    procs = [ctx.Process(target=_shard_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][3] == [0, 4] and res[1][3] == [4, 8]
    for _, got, full, _ in res:
        assert got == full
    from stac_b200.sharding import head_slice
    with pytest.raises(ValueError):
        head_slice(0, 3, 16)


def test_launch_state_is_kept_per_device(tmp_path):
    """The shared-memory opt-in of a kernel and the SM count belong to a GPU: the bookkeeping the
    launchers use (csrc/per_device.h, host-only C++) keeps one entry per device ordinal."""
    import subprocess
    src = tmp_path / "per_device_test.cpp"
    src.write_text('#include "per_device.h"\n'
                   "int main() {\n"
                   "  stac::PerDeviceFlag f;\n"
                   "  stac::PerDeviceValue<int> sm;\n"
                   "  if (!f.needs_setup(0) || !f.needs_setup(1)) return 1;\n"
                   "  f.mark(0);\n"
                   "  if (f.needs_setup(0)) return 2;\n"
                   "  if (!f.needs_setup(1)) return 3;          // device 1 still has to opt in\n"
                   "  sm.set(0, 148);\n"
                   "  if (sm.get(0) != 148 || sm.get(1) != 0) return 4;\n"
                   "  if (!stac::device_index_ok(63) || stac::device_index_ok(64) || stac::device_index_ok(-1)) return 5;\n"
                   "  return 0;\n"
                   "}\n")
    exe = tmp_path / "per_device_test"
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "stac_b200", "csrc"), str(src), "-o", str(exe)],
                   check=True)
    assert subprocess.run([str(exe)]).returncode == 0
    # no launcher keeps a process-wide "attribute already set" or SM-count static any more
    for name in ("attn_colsum.cu", "h2o.cu", "retrieve.cu", "voxel.cu"):
        text = open(os.path.join(ROOT, "stac_b200", "csrc", name)).read()
        assert not re.search(r"static\s+(bool|int)\s+(attr_done|attr_smem|n_sm)\b", text), name


def test_checkpoint_file_loads_without_pickle(tmp_path):
    """save_state / load_state round trip of a state dictionary with every value type the managers
    emit (tensors, lists, numbers, strings, None, nested dicts), read back with weights_only=True."""
    import torch
    from stac_b200.stac.checkpoint import load_state, save_state

    class Stub:
        device = torch.device("cpu")

        def __init__(self):
            self.loaded = None

        def state_dict(self):
            return {"format": 1, "class": "STACVoxelKV", "shape": [2, 3, 64, 21, 147], "use_cpu": False,
                    "key": torch.arange(12, dtype=torch.bfloat16).view(2, 3, 2), "key_cpu": None,
                    "offset_hot": [5, 5], "temperature": 0.9,
                    "memory": {"meta": torch.arange(8, dtype=torch.int32), "over": {"S": torch.zeros(0)},
                               "voxel_alloc": 64},
                    "retrieved": [torch.ones(2, 2), torch.zeros(2, dtype=torch.bool)]}

        def load_state_dict(self, sd):
            self.loaded = sd

    a, b = Stub(), Stub()
    path = str(tmp_path / "stream.pt")
    save_state(a, path)
    load_state(b, path)
    want = a.state_dict()
    assert b.loaded["offset_hot"] == want["offset_hot"] and b.loaded["key_cpu"] is None
    assert torch.equal(b.loaded["key"], want["key"]) and b.loaded["key"].dtype == torch.bfloat16
    assert torch.equal(b.loaded["memory"]["meta"], want["memory"]["meta"])
    assert b.loaded["retrieved"][1].dtype == torch.bool
