"""The remaining row-parallel launchers of the reference's gpu_ops module (src/gpu_ops.h:78-105,117): hyper-connection
norm / low-rank / mix, the PLE gate, the MTP concat and Mamba-2's gated group norm, against the oracle's statement of
the kernels (src/gpu_ops.hip:322-476, 762-792)."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import dev, host, max_rel_rows

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,hc,T", [(1024, 4, 9), (2560, 2, 5), (256, 4, 33), (4096, 3, 4)])
def test_hc_norm(ops, oracle, n, hc, T):
    res = synth.normal(0, "hc.r", 0, T * hc * n).reshape(T, hc, n)
    cur = synth.normal(0, "hc.c", 0, T * n).reshape(T, n)
    inj = synth.normal(0, "hc.i", 0, T * hc).reshape(T, hc) * 3
    w = synth.normal(0, "hc.w", 0, hc * n, 1.0, 0.1).reshape(hc, n)
    d_res, d_w = dev(res), dev(w)
    y, ro = torch.empty_like(d_res), torch.full_like(d_res, -3.0)
    ops.gpu_hc_norm(d_res, None, None, None, d_w, y, n, hc, T, 1e-6)          # the norm alone
    torch.cuda.synchronize()
    _, wy = oracle.hc_norm(res, None, None, w, hc, 1e-6)
    assert np.array_equal(host(y).view(np.uint32), wy.view(np.uint32))
    q8 = ops.Q8Buffers(T * hc * n, "cuda", xh="bf16")
    ops.gpu_hc_norm(d_res, ro, dev(cur), dev(inj), d_w, y, n, hc, T, 1e-6, q8=q8)
    torch.cuda.synchronize()
    wro, wy = oracle.hc_norm(res, cur, inj, w, hc, 1e-6)
    assert max_rel_rows(host(ro).reshape(-1, n), wro.reshape(-1, n)) <= 1e-6      # (expf differs by an ulp or two)
    _, wy2 = oracle.hc_norm(host(ro), None, None, w, hc, 1e-6)                     # the norm of what was stored: exact
    assert np.array_equal(host(y).view(np.uint32), wy2.view(np.uint32))
    assert max_rel_rows(host(y).reshape(-1, n), wy.reshape(-1, n)) <= 1e-5
    want = oracle.quantize_q8(host(y).reshape(-1), xh="bf16")
    for k in ("q0", "d0", "qK", "dK", "bsK"):
        assert np.array_equal(host(getattr(q8, k)).view(want[k].dtype), want[k]), k
    inplace = d_res.clone()
    ops.gpu_hc_norm(inplace, inplace, dev(cur), dev(inj), d_w, y, n, hc, T, 1e-6)  # res_out may be res_in
    torch.cuda.synchronize()
    assert torch.equal(inplace, ro)
    with pytest.raises(ops.LayerOpError):
        ops.gpu_hc_norm(d_res, ro, None, None, d_w, y, n + 4, hc, T, 1e-6)


@pytest.mark.parametrize("n,np_,T,hc", [(100, 128, 17, 4), (64, 64, 5, 2), (37, 96, 3, 4)])
def test_hc_lowrank(ops, oracle, n, np_, T, hc):
    lo = synth.normal(1, "lr.x", 0, T * n).reshape(T, n) * 4
    out = torch.full((T, np_), -1.0, device="cuda")
    ops.gpu_hc_lowrank(dev(lo), out, n, np_, T, hc)
    torch.cuda.synchronize()
    want = oracle.hc_lowrank(lo, np_, hc)
    assert np.abs(host(out) - want).max() <= 1e-6 * max(1.0, np.abs(want).max()) and not host(out)[:, n:].any()
    with pytest.raises(ops.LayerOpError):
        ops.gpu_hc_lowrank(dev(lo), out, n, n - 1, T, hc)


@pytest.mark.parametrize("n,hc,T", [(1024, 4, 11), (250, 3, 7), (256, 1, 4)])
def test_hc_mix(ops, oracle, n, hc, T):
    xn = synth.normal(2, "mx.x", 0, T * hc * n).reshape(T, hc, n)
    gate = synth.normal(2, "mx.g", 0, T * hc * n).reshape(T, hc, n) * 2
    out = torch.empty(T, n, device="cuda")
    ops.gpu_hc_mix(dev(xn), dev(gate), out, n, hc, T)
    torch.cuda.synchronize()
    assert max_rel_rows(host(out), oracle.hc_mix(xn, gate, hc)) <= 1e-6


@pytest.mark.parametrize("n,hc,T", [(1024, 4, 6), (768, 2, 9), (4096, 2, 3)])
def test_ple_gate(ops, oracle, n, hc, T):
    key = synth.normal(3, "pg.k", 0, T * hc * n).reshape(T, hc, n)
    res = synth.normal(3, "pg.r", 0, T * hc * n).reshape(T, hc, n)
    value = synth.normal(3, "pg.v", 0, T * n).reshape(T, n)
    res[0, 0] = -key[0, 0]                                # a clearly negative score
    res[1, 0] = key[1, 0]                                 # and a clearly positive one
    wk, wq, wc = (synth.normal(3, "pg.w%d" % i, 0, hc * n, 1.0, 0.1).reshape(hc, n) for i in range(3))
    gated, normed = torch.empty(T, hc, n, device="cuda"), torch.empty(T, hc, n, device="cuda")
    ops.gpu_ple_gate(dev(key), dev(value), dev(res), dev(wk), dev(wq), dev(wc), gated, normed, n, hc, T, 1e-6)
    torch.cuda.synchronize()
    wg, wn = oracle.ple_gate(key, value, res, wk, wq, wc, 1e-6)
    assert max_rel_rows(host(gated).reshape(-1, n), wg.reshape(-1, n)) <= 1e-5
    assert max_rel_rows(host(normed).reshape(-1, n), wn.reshape(-1, n)) <= 1e-5
    g = host(gated)[:, :, 0] / value[:, None, 0]
    assert g[0, 0] < 0.5 < g[1, 0]


@pytest.mark.parametrize("n,hc,T", [(512, 4, 7), (50, 2, 3)])
def test_mtp_concat(ops, n, hc, T):
    e = synth.normal(4, "mc.e", 0, T * n).reshape(T, n)
    h = synth.normal(4, "mc.h", 0, T * hc * n).reshape(T, hc, n)
    out = torch.empty(T, hc, 2 * n, device="cuda")
    ops.gpu_mtp_concat(dev(e), dev(h), out, n, hc, T)
    torch.cuda.synchronize()
    want = np.concatenate([np.broadcast_to(e[:, None, :], (T, hc, n)), h], axis=2)
    assert np.array_equal(host(out), want)


@pytest.mark.parametrize("d_inner,n_group,T", [(4096, 8, 5), (2048, 2, 9), (768, 1, 4), (1024, 4, 3)])
def test_mamba_gnorm(ops, oracle, d_inner, n_group, T):
    ld = d_inner + 2 * 128 + 64                           # [z d_inner | xBC | dt] rows
    y = synth.normal(5, "gn.y", 0, T * d_inner).reshape(T, d_inner)
    zx = synth.normal(5, "gn.z", 0, T * ld).reshape(T, ld) * 2
    w = synth.normal(5, "gn.w", 0, d_inner, 1.0, 0.1)
    out = torch.empty(T, d_inner, device="cuda")
    q8 = ops.Q8Buffers(T * d_inner, "cuda") if (T * d_inner) % 256 == 0 else None
    ops.gpu_mamba_gnorm(dev(y), dev(zx), ld, dev(w), out, d_inner, n_group, T, 1e-5, q8=q8)
    torch.cuda.synchronize()
    assert max_rel_rows(host(out), oracle.mamba_gnorm(y, zx[:, :d_inner], w, n_group, 1e-5)) <= 1e-5
    if q8 is not None:
        want = oracle.quantize_q8(host(out).reshape(-1))
        assert np.array_equal(host(q8.q0).view(np.int8), want["q0"]) and np.array_equal(host(q8.qK).view(np.int8), want["qK"])
    with pytest.raises(ops.LayerOpError):
        ops.gpu_mamba_gnorm(dev(y), dev(zx), ld, dev(w), out, d_inner, 5, T, 1e-5)       # d_inner % n_group != 0
