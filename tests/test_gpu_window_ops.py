"""The launchers that look back over earlier tokens (src/gpu_ops.h:96-116): Mamba-2 conv and selective scan, the PLE
conv, against the oracle's statement of the kernels (src/gpu_ops.hip:476-512, 679-760); and a batch processed in two
halves gives the bits of the whole batch (the carried state is the only coupling)."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import dev, host, max_rel_rows

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("conv_dim,d_conv,T,x_off,extra", [(1024, 4, 37, 512, 64), (640, 2, 5, 128, 16), (100, 8, 3, 7, 5),
                                                            (256, 4, 2, 0, 0)])
def test_mamba_conv(ops, oracle, conv_dim, d_conv, T, x_off, extra):
    ld = x_off + conv_dim + extra
    zx = synth.normal(0, "mv.z", 0, T * ld).reshape(T, ld)
    st = synth.normal(0, "mv.s", 0, conv_dim * (d_conv - 1)).reshape(conv_dim, d_conv - 1)
    w = synth.normal(0, "mv.w", 0, conv_dim * d_conv, 0.0, 0.5).reshape(conv_dim, d_conv)
    b = synth.normal(0, "mv.b", 0, conv_dim, 0.0, 0.1)
    d_st, out = dev(st), torch.empty(T, conv_dim, device="cuda")
    ops.gpu_mamba_conv(dev(zx), ld, x_off, d_st, dev(w), dev(b), out, conv_dim, d_conv, T)
    torch.cuda.synchronize()
    want, wst = oracle.mamba_conv(zx, x_off, st, w, b, conv_dim, d_conv)
    assert max_rel_rows(host(out), want) <= 1e-6
    assert np.array_equal(host(d_st), wst)
    # two halves with the carried state: the same bits as the whole batch
    if T >= 2:
        h = T // 2
        d_st2, o2 = dev(st), torch.empty(T, conv_dim, device="cuda")
        dz = dev(zx)
        ops.gpu_mamba_conv(dz, ld, x_off, d_st2, dev(w), dev(b), o2, conv_dim, d_conv, h)
        ops.gpu_mamba_conv(dz[h:], ld, x_off, d_st2, dev(w), dev(b), o2[h:], conv_dim, d_conv, T - h)
        torch.cuda.synchronize()
        assert torch.equal(o2, out) and torch.equal(d_st2, d_st)
    with pytest.raises(ops.LayerOpError):
        ops.gpu_mamba_conv(dev(zx), ld, x_off, d_st, dev(w), dev(b), out, conv_dim, 9, T)


@pytest.mark.parametrize("m,K,dil,T", [(512, 4, 2, 19), (100, 3, 1, 7), (256, 2, 3, 2), (64, 1, 1, 5), (128, 4, 4, 3)])
def test_ple_conv(ops, oracle, m, K, dil, T):
    H = (K - 1) * dil
    normed = synth.normal(1, "pc.n", 0, T * m).reshape(T, m)
    gated = synth.normal(1, "pc.g", 0, T * m).reshape(T, m)
    res = synth.normal(1, "pc.r", 0, T * m).reshape(T, m)
    st = synth.normal(1, "pc.s", 0, max(H, 1) * m).reshape(max(H, 1), m)[:H]
    wb = oracle.f32_to_f16(synth.normal(1, "pc.w", 0, m * K, 0.0, 0.5)).reshape(m, K)
    d_res, d_st = dev(res), dev(st) if H else None
    mids = [torch.full((max(H, 1), m), -9.0, device="cuda") for _ in range(3)] if H else None
    ops.gpu_ple_conv(dev(normed), dev(gated), d_res, d_st, dev(wb, torch.float16), m, T, K, dil, state_mid=mids)
    torch.cuda.synchronize()
    wres, wst, wmid = oracle.ple_conv(normed, gated, res, st, wb, K, dil, n_mid=3)
    assert max_rel_rows(host(d_res), wres) <= 1e-6
    if H:
        assert np.array_equal(host(d_st), wst)
        for j in range(3):
            if j < T - 1:
                assert np.array_equal(host(mids[j]), wmid[j]), j
            else:
                assert (host(mids[j]) == -9.0).all()
        # a rollback point is the state a shorter batch leaves: process j + 1 tokens only
        if T >= 3:
            s2, r2 = dev(st), dev(res)
            ops.gpu_ple_conv(dev(normed), dev(gated), r2, s2, dev(wb, torch.float16), m, 2, K, dil)
            torch.cuda.synchronize()
            assert torch.equal(s2, mids[1])


@pytest.mark.parametrize("n_head,n_group,T", [(8, 2, 9), (16, 1, 4), (4, 4, 17)])
def test_mamba_scan(ops, oracle, n_head, n_group, T):
    d_inner = n_head * 64
    conv_dim = d_inner + 2 * n_group * 128
    dt_off = d_inner + conv_dim
    ld = dt_off + n_head
    xbc = synth.normal(2, "ms.x", 0, T * conv_dim).reshape(T, conv_dim)
    zx = synth.normal(2, "ms.z", 0, T * ld).reshape(T, ld)
    zx[0, dt_off] = 25.0                                   # softplus's pass-through branch
    state = synth.normal(2, "ms.s", 0, n_head * 64 * 128).reshape(n_head, 64, 128) * 0.1
    dt_b = synth.normal(2, "ms.b", 0, n_head, 0.0, 0.5)
    A = -np.abs(synth.normal(2, "ms.a", 0, n_head, 1.0, 0.3)).astype(np.float32)
    D = synth.normal(2, "ms.d", 0, n_head, 1.0, 0.1)
    d_state, y = dev(state), torch.empty(T, d_inner, device="cuda")
    ops.gpu_mamba_scan(d_state, dev(xbc), dev(zx), ld, dt_off, dev(dt_b), dev(A), dev(D), y, n_head, d_inner, n_group, T)
    torch.cuda.synchronize()
    wy, ws = oracle.mamba_scan(state, xbc, zx, dt_off, dt_b, A, D, n_head, n_group)
    assert max_rel_rows(host(y), wy) <= 1e-5
    assert max_rel_rows(host(d_state).reshape(n_head * 64, 128), ws.reshape(n_head * 64, 128)) <= 1e-5
    # two halves with the carried state: the same bits
    h = T // 2
    s2, y2 = dev(state), torch.empty(T, d_inner, device="cuda")
    dx, dz = dev(xbc), dev(zx)
    ops.gpu_mamba_scan(s2, dx, dz, ld, dt_off, dev(dt_b), dev(A), dev(D), y2, n_head, d_inner, n_group, h)
    ops.gpu_mamba_scan(s2, dx[h:], dz[h:], ld, dt_off, dev(dt_b), dev(A), dev(D), y2[h:], n_head, d_inner, n_group, T - h)
    torch.cuda.synchronize()
    assert torch.equal(y2, y) and torch.equal(s2, d_state)
    with pytest.raises(ops.LayerOpError):
        ops.gpu_mamba_scan(d_state, dx, dz, ld, dt_off, dev(dt_b), dev(A), dev(D), y, n_head, d_inner + 64, n_group, T)
