"""Generate ``attention_ref.npz`` by running the reference's OWN attention kernels on a GPU.

The reference's window + pivot attention exists only as GPU code; its Triton entry point
``fa_forward_colsum_fast_sub`` (stac/flash_attn_triton.py:900-1006, kernels :21-125 and
:435-513) is the one that runs without building an extension.  This script feeds it the seeded
inputs of ``cases.ATTENTION_REF`` and stores what it returns: O (bf16 bits), lse and the
per-key column sums (fp32), plus its time per call for the largest case.

    python oracle/make_ref.py /path/to/reference        # stages the sources, git-ignored
    python tests/golden/make_attention_ref.py [out.npz] # on a machine with a CUDA GPU

Only the outputs are stored; the tests rebuild the inputs from the seeds.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def main(out_path):
    import torch
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isfile(os.path.join(ref_dir, "stac", "flash_attn_triton.py")):
        sys.exit("oracle/_ref is missing: run `python oracle/make_ref.py /path/to/reference` first")
    sys.path.insert(0, ref_dir)
    from stac.flash_attn_triton import fa_forward_colsum_fast_sub
    dev = torch.device("cuda:0")
    out = {}
    for name, c in cases.ATTENTION_REF.items():
        q, k, v, bias = cases.attention_inputs(name)
        tq = torch.from_numpy(q).to(dev, torch.bfloat16).unsqueeze(0)      # [1,M,H,D]
        tk = torch.from_numpy(k).to(dev, torch.bfloat16).unsqueeze(0)      # [1,N,H,D]
        tv = torch.from_numpy(v).to(dev, torch.bfloat16).unsqueeze(0)
        tb = None
        if bias is not None:
            tb = torch.from_numpy(bias).to(dev).view(1, c["H"], 1, c["N"])  # the manager's layout
        o, lse, cs = fa_forward_colsum_fast_sub(tq, tk, tv, bias=tb, write_o=True,
                                                subsample_ratio=c["ratio"])
        torch.cuda.synchronize()
        out[f"{name}_out_bf16"] = o[0].contiguous().view(torch.int16).cpu().numpy()   # [M,H,D] raw bits
        out[f"{name}_lse"] = lse[0, :, :c["M"]].float().cpu().numpy()                # [H,M]
        out[f"{name}_colsum"] = cs[0].float().cpu().numpy()                           # [H,N]
        assert np.isfinite(out[f"{name}_colsum"]).all(), name
    # time of the reference kernel pair at the microbenchmark and stream shapes, for the record
    # (random inputs; a same-device comparator, not a fixture)
    def timed(M, N, H=16):
        g = torch.Generator(device=dev).manual_seed(0)
        tq = (torch.randn(1, M, H, 64, device=dev, generator=g) / 8).to(torch.bfloat16)
        tk = (torch.randn(1, N, H, 64, device=dev, generator=g) / 8).to(torch.bfloat16)
        tv = (torch.randn(1, N, H, 64, device=dev, generator=g) / 8).to(torch.bfloat16)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            fa_forward_colsum_fast_sub(tq, tk, tv, bias=None, write_o=True, subsample_ratio=1.0)
        ev0.record()
        for _ in range(10):
            fa_forward_colsum_fast_sub(tq, tk, tv, bias=None, write_o=True, subsample_ratio=1.0)
        ev1.record()
        torch.cuda.synchronize()
        return ev0.elapsed_time(ev1) / 10

    shapes = [(1041, 2082), (1041, 10376), (1041, 33312), (4164, 17697)]
    out["meta_timed_shapes_M_N"] = np.array(shapes, np.int64)
    out["meta_timed_ms"] = np.array([timed(M, N) for M, N in shapes], np.float32)
    out["meta_gpu"] = np.array(torch.cuda.get_device_name(0))
    out["meta_torch_triton"] = np.array(f"torch {torch.__version__}, triton {__import__('triton').__version__}")
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, "reference Triton ms per call at", shapes, "=", out["meta_timed_ms"].tolist())


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "attention_ref.npz"))
