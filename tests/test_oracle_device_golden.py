"""The CPU checkers against the REFERENCE'S OWN device kernels (src/gpu_ops.hip with src/q8_device.h, launched by
src/gpu_ops.cpp), whose inputs and outputs tests/golden/device_ops.npz holds: those files were compiled unchanged
against a host SIMT emulation (oracle/simt/) and run on the CPU by tests/golden/make_golden_device.py.

Two bars. The int8 side outputs (Q8_0 / Q8_K values, scales, sums, the 16-bit copy) are integer and byte work: the
restatement applied to the reference's own finished vector must give the reference's bytes. The fp32 outputs differ
between the reference's kernels (fp32 sums of squares in its block-reduction order) and the checkers (sums in double,
as the reference's CPU code and this build's kernels keep them) by the rounding of one fp32 sum: 2e-6 relative to the
row's largest magnitude; ops without a reduction are held to a few units in the last place of the transcendental.
"""
import os

import numpy as np
import pytest

from oracle import oracle

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "device_ops.npz"))
SIDE = ("q0", "d0", "s0", "qK", "dK", "bsK", "xh")


def close_rows(got, want, tol=2e-6):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape
    scale = np.abs(want).reshape(want.shape[0], -1).max(axis=1).reshape((-1,) + (1,) * (want.ndim - 1))
    assert np.all(np.abs(got - want) <= tol * np.maximum(scale, 1e-30)), float(np.abs(got - want).max())


def side_equal(tag, y, K, xh_kind):
    """Restated quantiser on the reference's finished vector y (first K values) == the reference's side outputs."""
    o = oracle.quantize_q8(np.ascontiguousarray(y.ravel()[:K]), xh=xh_kind, int8=True)
    for k in SIDE:
        want = G[f"{tag}_{k}"]
        assert np.array_equal(o[k].view(want.dtype), want[:o[k].size]), (tag, k)


@pytest.mark.parametrize("tag,add", [("rows", True), ("rows_noadd", False), ("split", True), ("odd", True)])
def test_add_rmsnorm_matches_the_reference_kernels(tag, add):
    x, w, y = G[f"norm_{tag}_x"], G[f"norm_{tag}_w"], G[f"norm_{tag}_y"]
    a = G[f"norm_{tag}_a"] if add else None
    xo, yo = oracle.add_rmsnorm(x, a, w, 1e-6)
    if add:
        assert np.array_equal(xo, G[f"norm_{tag}_xo"])        # one fp32 add: bit-exact
    close_rows(yo, y)
    if f"norm_{tag}_q0" in G:
        side_equal(f"norm_{tag}", y, y.size, "bf16")


@pytest.mark.parametrize("tag", ["full", "tail"])
def test_swiglu_matches_the_reference_kernel(tag):
    g, u, out = G[f"swiglu_{tag}_g"], G[f"swiglu_{tag}_u"], G[f"swiglu_{tag}_out"]
    got = oracle.swiglu(g, u)
    assert np.all(np.abs(got - out) <= 4e-7 * np.maximum(np.abs(out), 1e-30) + 1e-38)   # __expf: the libm expf here
    # the side outputs cover the values rounded up to whole Q8_K blocks, those past n taken as 0
    n = out.size
    K = (n + 255) // 256 * 256
    padded = np.zeros(K, np.float32)
    padded[:n] = out
    o = oracle.quantize_q8(padded, xh="f16", int8=True)
    for k in SIDE:
        want = G[f"swiglu_{tag}_{k}"]
        m = min(o[k].size, n if k in ("q0", "qK", "xh") else o[k].size)
        assert np.array_equal(o[k].view(want.dtype)[:m], want[:m]), (tag, k)


def test_quantiser_rules_on_exact_inputs():
    """relu2 of values whose squares are exact: the output is known to the bit, so this pins the quantiser alone."""
    x, out = G["relu2_x"], G["relu2_out"]
    assert np.array_equal(oracle.relu2(x), out)
    side_equal("relu2", out, out.size, "bf16")
    assert np.all(G["relu2_q0"].reshape(2, -1)[0, 32:64] == 0) and G["relu2_d0"][1] == 0     # the all-zero block


def test_gemma_chains_match_the_reference_kernels():
    eps = 1e-6
    close_rows(oracle.add_normed(G["add_normed_base"], G["add_normed_a"], G["add_normed_w"], G["add_normed_scale"][0], eps),
               G["add_normed_out"])
    xo, y1, y2 = oracle.gemma_attn_post(G["attn_post_x"], G["attn_post_a"], G["attn_post_wa"], G["attn_post_w1"],
                                        G["attn_post_w2"], eps)
    close_rows(xo, G["attn_post_xo"])
    close_rows(y1, G["attn_post_y1"], 4e-6)
    close_rows(y2, G["attn_post_y2"], 4e-6)
    xo, y = oracle.gemma_ffn_post(G["ffn_post_x"], G["ffn_post_mlp"], G["ffn_post_down"], G["ffn_post_wts"], G["ffn_post_ids"],
                                  G["ffn_post_es"], G["ffn_post_w1"], G["ffn_post_w2"], G["ffn_post_wp"],
                                  G["ffn_post_scale"][0], G["ffn_post_wn"], eps)
    close_rows(xo, G["ffn_post_xo"], 4e-6)
    close_rows(y, G["ffn_post_y"], 6e-6)


def test_combine_geglu_softcap_match_the_reference_kernels():
    got = oracle.moe_combine(G["ffn_post_down"], G["ffn_post_wts"], G["combine_shared"], G["combine_sg"], G["ffn_post_ids"],
                             G["ffn_post_es"])
    assert np.array_equal(got, G["combine_out"])                  # products and adds in slot order: bit-exact
    gu = G["geglu_gu"]
    n = gu.shape[1] // 2
    got = oracle.geglu(gu[:, :n], gu[:, n:])
    close_rows(got, G["geglu_out"], 1e-6)                          # tanhf of the libm against the rounded tanh
    got = oracle.softcap(G["softcap_x"], 30.0)
    assert np.all(np.abs(got - G["softcap_out"]) <= 4e-6 * 30.0)


def test_hyper_connection_and_ple_ops_match_the_reference_kernels():
    ro, y = oracle.hc_norm(G["hc_res"], G["hc_cur"], G["hc_inj"], G["hc_w"], 2, 1e-6)
    n = y.shape[-1]
    close_rows(ro.reshape(-1, n), G["hc_res_out"].reshape(-1, n))
    close_rows(y.reshape(-1, n), G["hc_y"].reshape(-1, n), 4e-6)
    side_equal("hc", G["hc_y"], G["hc_y"].size, "bf16")
    want = G["lowrank_out"]
    got = oracle.hc_lowrank(G["lowrank_lo"], want.shape[1], 4)
    assert np.abs(got - want).max() <= 1e-6 * max(1.0, np.abs(want).max()) and not want[:, 100:].any()
    close_rows(oracle.hc_mix(G["mix_xn"], G["mix_gate"], 2), G["mix_out"], 1e-6)
    g, nm = oracle.ple_gate(G["ple_key"], G["ple_val"], G["ple_res"], G["ple_wk"], G["ple_wq"], G["ple_wc"], 1e-6)
    close_rows(g.reshape(-1, n), G["ple_gated"].reshape(-1, n), 1e-5)
    close_rows(nm.reshape(-1, n), G["ple_normed"].reshape(-1, n), 1e-5)
    e, h = G["mtp_e"], G["mtp_h"]
    assert np.array_equal(G["mtp_out"], np.concatenate([np.broadcast_to(e[:, None, :], h.shape), h], axis=2))
    res, st, mids = oracle.ple_conv(G["pconv_normed"], G["pconv_gated"], G["pconv_res"], G["pconv_state"], G["pconv_w"], 4, 2, n_mid=3)
    close_rows(res, G["pconv_res_out"], 1e-6)
    assert np.array_equal(st, G["pconv_state_out"])
    for j in range(3):
        assert np.array_equal(mids[j], G["pconv_mid"][j]), j


def test_mamba_ops_match_the_reference_kernels():
    zx = G["gnorm_zx"]
    d_inner = G["gnorm_y"].shape[1]
    close_rows(oracle.mamba_gnorm(G["gnorm_y"], zx[:, :d_inner], G["gnorm_w"], 2, 1e-5), G["gnorm_out"], 4e-6)
    conv_dim, d_conv = G["conv_w"].shape
    out, st = oracle.mamba_conv(G["conv_zx"], 64, G["conv_state"], G["conv_w"], G["conv_bias"], conv_dim, d_conv)
    close_rows(out, G["conv_out"], 1e-6)
    assert np.array_equal(st, G["conv_state_out"])
    n_head = G["scan_A"].size
    dt_off = n_head * 64 + G["scan_xbc"].shape[1]
    y, s = oracle.mamba_scan(G["scan_state"], G["scan_xbc"], G["scan_zx"], dt_off, G["scan_dtb"], G["scan_A"], G["scan_D"], n_head, 2)
    close_rows(y, G["scan_y"], 1e-5)
    close_rows(s.reshape(-1, 128), G["scan_state_out"].reshape(-1, 128), 1e-5)


def test_routers_and_grouping_match_the_reference_kernels():
    nu = G["router_ids"].shape[1]
    ids, wts, sg = oracle.moe_router(G["router_logits"], nu, G["router_x"], G["router_w"])
    assert np.array_equal(ids, G["router_ids"])                       # selection: exact, ties to the lower index
    assert np.abs(wts - G["router_wts"]).max() <= 1e-6 and np.abs(sg - G["router_sg"]).max() <= 2e-6
    ids2, wts2 = oracle.moe_router_sigmoid(G["router_logits"], G["sigrouter_bias"], nu, 1, 2.5)
    assert np.array_equal(ids2, G["sigrouter_ids"]) and np.abs(wts2 - G["sigrouter_wts"]).max() <= 5e-6
    # grouping: entries by expert, runs cut into tiles; inside a run the reference's order is whatever its atomics gave
    ids, tile = G["router_ids"], int(G["group_tile"][0])
    flat = ids.ravel()
    counts = np.bincount(flat, minlength=64)
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    te = [e for e in range(64) for _ in range(0, counts[e], tile)]
    ts = [starts[e] + k for e in range(64) for k in range(0, counts[e], tile)]
    tn = [min(tile, counts[e] - k) for e in range(64) for k in range(0, counts[e], tile)]
    k = int(G["group_n_tiles"][0])
    assert k == len(te)
    assert np.array_equal(G["group_tile_e"][:k], te) and np.array_equal(G["group_tile_start"][:k], ts)
    assert np.array_equal(G["group_tile_n"][:k], tn)
    pair = G["group_pair"]
    assert np.array_equal(np.sort(pair), np.arange(flat.size)) and np.array_equal(flat[pair], np.sort(flat))
    assert np.array_equal(G["group_tok"], pair // nu)


def _prep(tag):
    D, nq, nkv, T, chain, gated, kvq, pos0, kv_stride = (int(v) for v in G[f"prep_{tag}_cfg"])
    rows = lambda a: a.reshape(-1, kv_stride)[pos0:pos0 + T]
    untouched = lambda a: (np.delete(a.reshape(-1, kv_stride), np.s_[pos0:pos0 + T], axis=0) == 0x5A5A).all()
    return D, nq, nkv, T, gated, kvq, pos0, rows, untouched


def _split_rows(r, n_vals, kq):
    """(value bytes, fp16 scale bits) of quantised cache rows given as uint16 [T][kv_stride] (src/attention.hip:44-55)."""
    b = np.ascontiguousarray(r).view(np.uint8)
    vb = n_vals if kq == 1 else n_vals // 2
    return b[:, :vb], b[:, vb:vb + n_vals // 16].copy().view(np.uint16)


@pytest.mark.parametrize("tag", ["exact_q8", "exact_q4", "exact_q8_rot", "exact_q4_rot", "exact_q8_rot512"])
def test_cache_rows_of_attn_prep_byte_for_byte(tag):
    """Norm and RoPE off: the reference's stored bytes follow from the inputs by exactly rounded steps, and the
    restated rotation (hadamard_rot) and quantiser (kv_quant_rows) must give the same bytes."""
    D, nq, nkv, T, gated, kvq, pos0, rows, untouched = _prep(tag)
    q, k, v = G[f"prep_{tag}_q"], G[f"prep_{tag}_k"], G[f"prep_{tag}_v"]
    rot, kq, n_vals = kvq & 4, kvq & 3, nkv * D
    N = oracle.hadamard_k(D)
    wq = oracle.hadamard_rot(q.reshape(-1, D), N).reshape(q.shape) if rot else q
    assert np.array_equal(G[f"prep_{tag}_q_out"], wq)
    wk = oracle.hadamard_rot(k.reshape(-1, D), N).reshape(k.shape) if rot else k
    wv = oracle.hadamard_rot(v.reshape(-1, D), 64).reshape(v.shape) if rot else v
    for name, want in (("K", wk), ("V", wv)):
        vals, scales = _split_rows(rows(G[f"prep_{tag}_{name}"]), n_vals, kq)
        want_q, want_d = oracle.kv_quant_rows(want, kq)
        assert np.array_equal(vals, want_q.view(np.uint8)), (tag, name)
        assert np.array_equal(scales, want_d), (tag, name)
        assert untouched(G[f"prep_{tag}_{name}"])


@pytest.mark.parametrize("tag", ["chain_f16", "chain_gated_f16", "chain_q8_rot", "chain_q4_rot"])
def test_attn_prep_chain_against_the_reference_kernel(tag):
    """Norm + RoPE (+ rotation, + quantisation): the reference's kernel sums squares in fp32 and takes powf / sincosf
    of the device library; the checker follows the reference's CPU code. q within 1e-5 of the row's largest
    magnitude, FP16 rows within one fp16 step, quantised rows within one quantisation step after decoding."""
    D, nq, nkv, T, gated, kvq, pos0, rows, untouched = _prep(tag)
    q, k, v = G[f"prep_{tag}_q"], G[f"prep_{tag}_k"], G[f"prep_{tag}_v"]
    rot, kq, n_vals = kvq & 4, kvq & 3, nkv * D
    wq, wk = oracle.qk_norm_rope(q, k, G[f"prep_{tag}_qn"], G[f"prep_{tag}_kn"], nq, nkv, D, D, 0, None, pos0, 1e6, 1e-6, gated=gated)
    wv = v
    if rot:
        N = oracle.hadamard_k(D)
        wq, wk = (oracle.hadamard_rot(a.reshape(-1, D), N).reshape(a.shape) for a in (wq, wk))
        wv = oracle.hadamard_rot(v.reshape(-1, D), 64).reshape(v.shape)
    close_rows(G[f"prep_{tag}_q_out"].reshape(-1, D), wq.reshape(-1, D), 1e-5)
    for name, want in (("K", wk), ("V", wv)):
        r = rows(G[f"prep_{tag}_{name}"])
        if kq == 0:
            got = oracle.f16_to_f32(r).reshape(want.shape)
            assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -10 + 1e-7), (tag, name)
        else:
            vals, scales = _split_rows(r, n_vals, kq)
            d = oracle.f16_to_f32(scales).reshape(T, n_vals // 32, 1)
            if kq == 1:
                dec = vals.view(np.int8).astype(np.float32).reshape(T, n_vals // 32, 32) * d
            else:
                nib = np.stack([vals & 15, vals >> 4], axis=-1).reshape(T, n_vals // 8, 4, 2)   # byte 4 j + k: values 8 j + k, 8 j + k + 4
                dec = (nib.transpose(0, 1, 3, 2).reshape(T, n_vals // 32, 32).astype(np.float32) - 8) * d
            # half a step of rounding, plus the scale's own fp16 rounding on up to 127 (8) steps; Q4_0 also clips
            # the one value at +8 steps to +7
            step = np.abs(d) * (0.57 if kq == 1 else 1.01) + 1e-6
            assert np.all(np.abs(dec - want.reshape(T, n_vals // 32, 32)) <= step), (tag, name)
        assert untouched(G[f"prep_{tag}_{name}"])


def test_attn_prep_at_the_position_the_reference_tests():
    """tests/forward_verify.cpp:835-853,903-906 compares the reference's attn_prep kernel with its CPU ops at position
    2499 to 1e-3, because the kernel forms the angles in fp32 where the CPU code (and this build) forms them in double:
    the same comparison here, the reference's kernel against the checker that follows its CPU code (measured: 6e-5)."""
    tag = "chain_pos2499"
    D, nq, nkv, T, gated, kvq, pos0, rows, untouched = _prep(tag)
    assert pos0 == 2499
    wq, wk = oracle.qk_norm_rope(G[f"prep_{tag}_q"], G[f"prep_{tag}_k"], G[f"prep_{tag}_qn"], G[f"prep_{tag}_kn"], nq, nkv, D, D, 0,
                                 None, pos0, 1e6, 1e-6)
    close_rows(G[f"prep_{tag}_q_out"].reshape(-1, D), wq.reshape(-1, D), 1e-3)
    close_rows(oracle.f16_to_f32(rows(G[f"prep_{tag}_K"])).reshape(-1, D), wk.reshape(-1, D), 2e-3)
    assert untouched(G[f"prep_{tag}_K"]) and untouched(G[f"prep_{tag}_V"])


def _f16_ulps(a, b):
    k = lambda u: np.where(u.astype(np.int32) & 0x8000, -(u.astype(np.int32) & 0x7FFF), u.astype(np.int32))
    return int(np.abs(k(a) - k(b)).max())


def test_fp16_component_kernels_on_their_test_programs_inputs():
    """The reference's "rmsnorm" and "rope_rotate_half" kernels (src/layernorm.hip, src/rope_embedding.hip) on the
    sweeps of its own test programs: the checkers restate those programs' CPU loops (a sequential fp32 sum where the
    kernel sums 32 strided partials), so the norm agrees to one fp16 step and the rotation to the bit; both pass the
    programs' rule (tests/layernorm_verify.cpp:40-43)."""
    bad = lambda g, r: np.abs(g - r) > 0.01 * np.maximum(np.abs(g), np.abs(r)) + 1e-4
    for t, e in ((8, 17), (32, 64), (5, 4096), (1, 96), (7, 48)):
        x, gam = G[f"p3norm_{t}x{e}_x"], G[f"p3norm_{t}x{e}_gamma"]
        for got, want in ((oracle.rmsnorm_f16(x, gam, 1e-5), G[f"p3norm_{t}x{e}_y"]),
                          (oracle.rmsnorm_f16(x, None, 1e-5), G[f"p3norm_{t}x{e}_y_nogamma"])):
            assert _f16_ulps(got, want) <= 1
            assert not bad(oracle.f16_to_f32(got), oracle.f16_to_f32(want)).any()
    for r, d in ((16, 16), (5, 32), (64, 128)):
        got = oracle.rope_rotate_half_f16(G[f"p3rope_{r}x{d}_x"], G[f"p3rope_{r}x{d}_c"], G[f"p3rope_{r}x{d}_s"])
        assert np.array_equal(got, G[f"p3rope_{r}x{d}_y"])


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(oracle.__file__), "_ref", "libref_emul.so")),
                    reason="the emulated reference kernels are built only where the reference's sources are present")
def test_fixtures_regenerate_identically(tmp_path, monkeypatch):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden_device", os.path.join(os.path.dirname(__file__), "golden",
                                                                                     "make_golden_device.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    monkeypatch.setattr(m, "OUT", str(tmp_path))
    m.main()
    new = np.load(os.path.join(str(tmp_path), "device_ops.npz"))
    assert sorted(new.files) == sorted(G.files)
    for k in G.files:
        if k in ("group_tok", "group_pair"):          # the order inside a run comes from atomics: not reproducible
            continue
        assert np.array_equal(new[k], G[k], equal_nan=True), k
