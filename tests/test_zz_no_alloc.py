"""The allocation-free attention entry point (stac_attn_colsum_noalloc) against the regular one.

Some embedders cannot call cudaMalloc when the hot loop runs (all device memory already
belongs to their own arena, or an allocation's device-wide synchronisation is not acceptable),
so this variant keeps its scratch in a fixed array inside the library.  The array is shared by
all calls and keeps old contents, hence two calls in a row with different shapes: the second
must not be disturbed by what the first left behind.  Collected last on purpose."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(M, H, T_hot, T_ret, seed):
    rs = np.random.RandomState(seed)
    D = 64
    f = lambda *s: torch.from_numpy(rs.randn(*s).astype(np.float32)).to(torch.bfloat16).to(DEV)
    bias = np.log(rs.randint(1, 9, size=(H, T_ret)).astype(np.float32))
    bias[rs.rand(H, T_ret) < 0.2] = -np.inf
    return f(M, H, D), f(H, T_hot, D), f(H, T_hot, D), f(H, T_ret, D), f(H, T_ret, D), torch.from_numpy(bias).to(DEV)


def _call_noalloc(q, kh, vh, kr, vr, bias, status):
    from stac_b200 import _lib
    from stac_b200._lib import ptr, stream_ptr
    M, H, D = q.shape
    T_hot, T_ret = kh.shape[1], kr.shape[1]
    out = torch.empty_like(q)
    lse = torch.empty((H, M), dtype=torch.float32, device=DEV)
    cs = torch.empty((H, T_hot + T_ret), dtype=torch.float32, device=DEV)
    rc = _lib.lib().stac_attn_colsum_noalloc(
        ptr(q), q.stride(0), ptr(kh), ptr(vh), kh.stride(1), kh.stride(0), T_hot, ptr(kr), ptr(vr), kr.stride(1),
        kr.stride(0), T_ret, ptr(bias), bias.stride(0), ptr(out), out.stride(0), ptr(lse), ptr(cs), cs.stride(0),
        M, H, D, 0.125, 1.0, ptr(status.word), stream_ptr())
    return rc, out, lse, cs


def _oracle(q, kh, vh, kr, vr, bias):
    from oracle.attention import attn_colsum as oracle_attn
    H, T_hot = kh.shape[0], kh.shape[1]
    k_all = torch.cat([kh, kr], 1).float().cpu().numpy().transpose(1, 0, 2)
    v_all = torch.cat([vh, vr], 1).float().cpu().numpy().transpose(1, 0, 2)
    b_all = np.concatenate([np.zeros((H, T_hot), np.float32), bias.cpu().numpy()], 1)
    return oracle_attn(q.float().cpu().numpy(), k_all, v_all, b_all)


# The third shape has 160 (head, key group) column-sum items, more than the 148 SMs: without a
# workspace the forward pass runs one CTA per item while the column-sum pass is cut evenly over
# the SMs and adds partial sums onto the zeros the forward pass left in the output.
SHAPES = [(700, 4, 900, 130, 7), (260, 2, 300, 70, 8), (300, 16, 3400, 140, 9)]


def test_noalloc_matches_oracle_and_workspace_entry_in_a_row():
    from stac_b200 import ops
    status = ops.DeviceStatus(torch.device(DEV))
    for M, H, T_hot, T_ret, seed in SHAPES:
        q, kh, vh, kr, vr, bias = _inputs(M, H, T_hot, T_ret, seed)
        rc, out, lse, cs = _call_noalloc(q, kh, vh, kr, vr, bias, status)
        assert rc == 0
        ref_out, ref_lse, ref_cs = ops.attn_colsum(q, kh, vh, T_hot, kr, vr, bias, T_ret, want_lse=True,
                                                   status=status)
        torch.cuda.synchronize()
        status.raise_if_set("attention")
        o_np, lse_np, cs_np = out.float().cpu().numpy(), lse.cpu().numpy(), cs.cpu().numpy()
        # against the existing entry point ...
        assert np.abs(o_np - ref_out.float().cpu().numpy()).max() <= 2e-2
        np.testing.assert_allclose(lse_np, ref_lse.cpu().numpy(), rtol=1e-3, atol=1e-3)
        np.testing.assert_allclose(cs_np, ref_cs.cpu().numpy(), rtol=1e-3, atol=1e-6)
        # ... and against the CPU oracle
        o_or, lse_or, cs_or = _oracle(q, kh, vh, kr, vr, bias)
        assert np.abs(o_np - o_or).max() <= 2e-2
        np.testing.assert_allclose(lse_np, lse_or, rtol=1e-3, atol=1e-3)
        np.testing.assert_allclose(cs_np, cs_or, rtol=1e-3, atol=1e-6)


def test_noalloc_rejects_oversize():
    from stac_b200 import _lib, ops
    status = ops.DeviceStatus(torch.device(DEV))
    q, kh, vh, kr, vr, bias = _inputs(64, 2, 128, 16, 1)
    M_big = 131072 // 2 + 1
    rc = _lib.lib().stac_attn_colsum_noalloc(
        _lib.ptr(q), q.stride(0), _lib.ptr(kh), _lib.ptr(vh), kh.stride(1), kh.stride(0), 128, None, None, 64, 64, 0,
        None, 0, _lib.ptr(q), q.stride(0), None, None, 0, M_big, 2, 64, 0.125, 1.0, _lib.ptr(status.word),
        _lib.stream_ptr())
    assert rc == 3
    assert _lib.lib().stac_status_string(rc) == b"capacity too small"
