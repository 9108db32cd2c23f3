"""This library's kernels on the inputs of tests/golden/device_ops.npz against the outputs the REFERENCE'S OWN device
kernels gave for them (src/gpu_ops.hip, src/attention.hip run through the host SIMT emulation of oracle/simt/; see
tests/golden/make_golden_device.py). Byte-exact where every step is exactly rounded (the quantisers on exact inputs,
cache rows, the rotation, combine, concat, selections, conv states); fp32 results of reductions within 2e-6 of the
row's largest magnitude (the reference's kernels sum squares in fp32, this library in double as the reference's CPU
code does), and int8 values computed from such results within one step."""
import os

import numpy as np
import pytest
import torch

from util import dev, host, max_rel_rows

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "device_ops.npz"))
SIDE = ("q0", "d0", "s0", "qK", "dK", "bsK", "xh")


def side_of(q8):
    return {k: host(getattr(q8, k)) for k in SIDE}


def test_quantisers_on_exact_inputs_give_the_reference_bytes(ops):
    x = G["relu2_x"]
    rows, h = x.shape
    out = torch.empty(rows, h, device="cuda")
    q8 = ops.Q8Buffers(rows * h, "cuda", xh="bf16")
    ops.gpu_relu2(dev(x), out, rows, h, h, q8=q8)
    torch.cuda.synchronize()
    assert np.array_equal(host(out), G["relu2_out"])
    for k, got in side_of(q8).items():
        want = G["relu2_" + k]
        assert np.array_equal(got.view(want.dtype), want[:got.size]), k


@pytest.mark.parametrize("tag,add", [("rows", True), ("rows_noadd", False), ("split", True), ("odd", True)])
def test_add_rmsnorm(ops, tag, add):
    x, w, want = G[f"norm_{tag}_x"], G[f"norm_{tag}_w"], G[f"norm_{tag}_y"]
    T, n = x.shape
    q8 = ops.Q8Buffers(T * n, "cuda", xh="bf16") if f"norm_{tag}_q0" in G else None
    xo, y = torch.empty(T, n, device="cuda"), torch.empty(T, n, device="cuda")
    ops.gpu_add_rmsnorm(dev(x), dev(G[f"norm_{tag}_a"]) if add else None, xo, dev(w), y, n, T, 1e-6, q8=q8)
    torch.cuda.synchronize()
    if add:
        assert np.array_equal(host(xo), G[f"norm_{tag}_xo"])
    assert max_rel_rows(host(y), want) <= 2e-6
    if q8 is not None:
        s = side_of(q8)
        for k in ("q0", "qK"):
            assert np.abs(s[k].view(np.int8).astype(np.int32) - G[f"norm_{tag}_{k}"][:T * n]).max() <= 1, k
        assert np.allclose(s["d0"], G[f"norm_{tag}_d0"][:T * n // 32], rtol=4e-6)
        assert np.allclose(s["dK"], G[f"norm_{tag}_dK"][:T * n // 256], rtol=4e-6)


@pytest.mark.parametrize("tag", ["full", "tail"])
def test_swiglu(ops, tag):
    g, u, want = G[f"swiglu_{tag}_g"], G[f"swiglu_{tag}_u"], G[f"swiglu_{tag}_out"]
    out = torch.empty(g.size, device="cuda")
    ops.gpu_swiglu(dev(g), dev(u), out, g.size)
    torch.cuda.synchronize()
    assert np.all(np.abs(host(out) - want) <= 4e-7 * np.abs(want) + 1e-38)


def test_gemma_chains(ops):
    T, n = G["add_normed_a"].shape
    out = torch.empty(T, n, device="cuda")
    ops.gpu_add_normed(dev(G["add_normed_base"]), dev(G["add_normed_a"]), dev(G["add_normed_w"]), dev(G["add_normed_scale"]), out,
                       n, T, 1e-6)
    xo, y1, y2 = (torch.empty(T, n, device="cuda") for _ in range(3))
    ops.gpu_gemma_attn_post(dev(G["attn_post_x"]), dev(G["attn_post_a"]), dev(G["attn_post_wa"]), xo, dev(G["attn_post_w1"]), y1,
                            dev(G["attn_post_w2"]), y2, n, T, 1e-6)
    fx, fy = torch.empty(T, n, device="cuda"), torch.empty(T, n, device="cuda")
    U = G["ffn_post_wts"].shape[1]
    ops.gpu_gemma_ffn_post(dev(G["ffn_post_x"]), dev(G["ffn_post_mlp"]), dev(G["ffn_post_down"]), dev(G["ffn_post_wts"]),
                           dev(G["ffn_post_ids"]), dev(G["ffn_post_es"]), U, dev(G["ffn_post_w1"]), dev(G["ffn_post_w2"]),
                           dev(G["ffn_post_wp"]), dev(G["ffn_post_scale"]), fx, dev(G["ffn_post_wn"]), fy, n, T, 1e-6)
    comb = torch.empty(T, n, device="cuda")
    ops.gpu_moe_combine(dev(G["ffn_post_down"]), dev(G["ffn_post_wts"]), dev(G["combine_shared"]), dev(G["combine_sg"]), comb, U,
                        n, T, ids=dev(G["ffn_post_ids"]), exp_scale=dev(G["ffn_post_es"]))
    torch.cuda.synchronize()
    assert max_rel_rows(host(out), G["add_normed_out"]) <= 2e-6
    assert max_rel_rows(host(xo), G["attn_post_xo"]) <= 2e-6
    assert max_rel_rows(host(y1), G["attn_post_y1"]) <= 4e-6 and max_rel_rows(host(y2), G["attn_post_y2"]) <= 4e-6
    assert max_rel_rows(host(fx), G["ffn_post_xo"]) <= 4e-6 and max_rel_rows(host(fy), G["ffn_post_y"]) <= 6e-6
    assert np.array_equal(host(comb), G["combine_out"])


def test_selections_and_exact_copies(ops):
    lg = G["router_logits"]
    T, ne = lg.shape
    nu = G["router_ids"].shape[1]
    ids = torch.zeros(T, nu, dtype=torch.int32, device="cuda")
    wts, sg = torch.zeros(T, nu, device="cuda"), torch.zeros(T, device="cuda")
    ops.gpu_moe_router(dev(lg), dev(G["router_x"]), dev(G["router_w"]), ids, wts, sg, ne, nu, G["router_x"].shape[1], T)
    ids2, wts2 = torch.zeros_like(ids), torch.zeros_like(wts)
    ops.gpu_moe_router_sigmoid(dev(lg), dev(G["sigrouter_bias"]), ids2, wts2, ne, nu, 1, 2.5, T)
    e, h = G["mtp_e"], G["mtp_h"]
    cat = torch.empty(*G["mtp_out"].shape, device="cuda")
    ops.gpu_mtp_concat(dev(e), dev(h), cat, e.shape[1], h.shape[1], e.shape[0])
    torch.cuda.synchronize()
    assert np.array_equal(host(ids), G["router_ids"]) and np.array_equal(host(ids2), G["sigrouter_ids"])
    assert np.abs(host(wts) - G["router_wts"]).max() <= 1e-6 and np.abs(host(sg) - G["router_sg"]).max() <= 2e-6
    assert np.abs(host(wts2) - G["sigrouter_wts"]).max() <= 5e-6
    assert np.array_equal(host(cat), G["mtp_out"])


@pytest.mark.parametrize("tag", ["exact_q8", "exact_q4", "exact_q8_rot", "exact_q4_rot", "exact_q8_rot512"])
def test_cache_rows_are_the_reference_kernels_bytes(ops, oracle, tag):
    D, nq, nkv, T, chain, gated, kvq, pos0, kv_stride = (int(v) for v in G[f"prep_{tag}_cfg"])
    rot, kq, n_vals = kvq & 4, kvq & 3, nkv * D
    N = oracle.hadamard_k(D)
    for name, src, blk in (("K", G[f"prep_{tag}_k"], N), ("V", G[f"prep_{tag}_v"], 64)):
        want = G[f"prep_{tag}_{name}"]
        cache = torch.full((want.size,), 0x5A5A, device="cuda", dtype=torch.int16)
        ops.gpu_kv_store_q(dev(src), cache, n_vals, None, pos0, T, kv_stride, 30, 0, kq, rot_block=blk if rot else 0)
        torch.cuda.synchronize()
        assert np.array_equal(cache.cpu().numpy().view(np.uint16), want), (tag, name)
    if rot:
        q = G[f"prep_{tag}_q"]
        out = torch.empty(T * nq, D, device="cuda")
        ops.gpu_hadamard_rot(dev(q.reshape(-1, D)), out, T * nq, D, N)
        torch.cuda.synchronize()
        assert np.array_equal(host(out).reshape(q.shape), G[f"prep_{tag}_q_out"])


@pytest.mark.parametrize("tag", ["chain_f16", "chain_gated_f16"])
def test_norm_rope_into_the_fp16_cache(ops, tag):
    D, nq, nkv, T, chain, gated, kvq, pos0, kv_stride = (int(v) for v in G[f"prep_{tag}_cfg"])
    q, k, v = G[f"prep_{tag}_q"], G[f"prep_{tag}_k"], G[f"prep_{tag}_v"]
    q_out = torch.empty(T, nq * D, device="cuda")
    K = torch.full((G[f"prep_{tag}_K"].size,), -3.0, device="cuda", dtype=torch.float16)
    V = torch.full_like(K, -3.0)
    ops.gpu_attn_prep_f16(dev(q), dev(k), dev(v), dev(G[f"prep_{tag}_qn"]), dev(G[f"prep_{tag}_kn"]), q_out, K, V, kv_stride, 30, 0,
                          nq, nkv, D, D, 0, None, pos0, T, 1e6, 1e-6, gated)
    torch.cuda.synchronize()
    assert max_rel_rows(host(q_out).reshape(-1, D), G[f"prep_{tag}_q_out"].reshape(-1, D)) <= 1e-5
    rows = lambda a: a.reshape(-1, kv_stride)[pos0:pos0 + T]
    for got, want in ((K, G[f"prep_{tag}_K"]), (V, G[f"prep_{tag}_V"])):
        a, b = host(got).view(np.float16).astype(np.float32), want.view(np.float16).astype(np.float32)
        assert np.all(np.abs(rows(a) - rows(b)) <= np.abs(rows(b)) * 2.0 ** -10 + 1e-7)


def test_fp16_component_kernels(ops):
    """gpu_rmsnorm_f16 / gpu_rope_rotate_half_f16 on the inputs of the reference's test programs against what the
    reference's own kernels gave (one fp16 step: the sums run in different orders)."""
    def ulps(a, b):
        k = lambda u: np.where(u.astype(np.int32) & 0x8000, -(u.astype(np.int32) & 0x7FFF), u.astype(np.int32))
        return int(np.abs(k(a) - k(b)).max())
    f16 = torch.float16
    for t, e in ((8, 17), (32, 64), (5, 4096), (1, 96), (7, 48)):
        x, gam = dev(G[f"p3norm_{t}x{e}_x"], f16), dev(G[f"p3norm_{t}x{e}_gamma"], f16)
        y = torch.empty_like(x)
        ops.gpu_rmsnorm_f16(x, gam, y, t, e, 1e-5)
        torch.cuda.synchronize()
        assert ulps(host(y), G[f"p3norm_{t}x{e}_y"]) <= 1
        ops.gpu_rmsnorm_f16(x, None, y, t, e, 1e-5)
        torch.cuda.synchronize()
        assert ulps(host(y), G[f"p3norm_{t}x{e}_y_nogamma"]) <= 1
    for r, d in ((16, 16), (5, 32), (64, 128)):
        x = dev(G[f"p3rope_{r}x{d}_x"], f16)
        y = torch.empty_like(x)
        ops.gpu_rope_rotate_half_f16(x, dev(G[f"p3rope_{r}x{d}_c"]), dev(G[f"p3rope_{r}x{d}_s"]), y, r, d // 2)
        torch.cuda.synchronize()
        assert ulps(host(y), G[f"p3rope_{r}x{d}_y"]) <= 1
