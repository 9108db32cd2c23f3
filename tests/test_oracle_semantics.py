"""Properties of the CPU restatement that the reference states in words or in its component tests: the fused
residual add, bf16 storage rules, partial rotary, the gated Q stride, and the two FP16 component-test references
replayed with the reference tests' own generator, shapes and pass rule."""
import numpy as np

from rocm_hip_b200 import synth


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_add_rmsnorm_is_add_then_norm(oracle):
    T, n = 5, 768
    x = synth.normal(0, "s.x", 0, T * n).reshape(T, n)
    a = synth.normal(0, "s.a", 0, T * n).reshape(T, n)
    w = synth.normal(0, "s.w", 0, n, 1.0, 0.1)
    xo, y = oracle.add_rmsnorm(x, a, w, 1e-6)
    assert np.array_equal(bits(xo), bits(x + a))
    _, y2 = oracle.add_rmsnorm(x + a, None, w, 1e-6)
    assert np.array_equal(bits(y), bits(y2))
    # definition check in float64
    v = (x + a).astype(np.float64)
    ref = v / np.sqrt((v * v).mean(axis=1, keepdims=True) + 1e-6) * w
    assert np.abs(y - ref).max() / np.abs(ref).max() < 1e-6


def test_bf16_fused_equals_unfused(oracle):
    T, n = 6, 512
    x = oracle.f32_to_bf16(synth.normal(0, "b.x", 0, T * n)).reshape(T, n)
    a = oracle.f32_to_bf16(synth.normal(0, "b.a", 0, T * n)).reshape(T, n)
    w = synth.normal(0, "b.w", 0, n, 1.0, 0.1)
    xo, y = oracle.add_rmsnorm_bf16(x, a, w, 1e-6)
    want_xo = oracle.f32_to_bf16(oracle.bf16_to_f32(x) + oracle.bf16_to_f32(a))
    assert np.array_equal(xo, want_xo)
    _, y2 = oracle.add_rmsnorm_bf16(xo, None, w, 1e-6)
    assert np.array_equal(y, y2)
    # and it is the fp32 op on the decoded stored sum, rounded once
    _, yf = oracle.add_rmsnorm(oracle.bf16_to_f32(xo), None, w, 1e-6)
    assert np.array_equal(y, oracle.f32_to_bf16(yf))


def test_partial_rotary_and_gated_stride(oracle):
    T, nq, nkv, D, n_rot = 4, 3, 2, 256, 64
    qf = synth.normal(0, "p.q", 0, T * nq * 2 * D).reshape(T, nq * 2 * D)  # [Q | gate] per head
    k = synth.normal(0, "p.k", 0, T * nkv * D).reshape(T, nkv * D)
    qn, kn = synth.normal(0, "p.qn", 0, D, 1.0, 0.1), synth.normal(0, "p.kn", 0, D, 1.0, 0.1)
    pos = np.array([0, 7, 2499, 100000], dtype=np.int32)
    qo, ko = oracle.qk_norm_rope(qf, k, qn, kn, nq, nkv, D, n_rot, 0, pos, 0, 1e7, 1e-6, gated=1)
    # the same through the ungated path on the compacted Q heads
    qc = qf.reshape(T, nq, 2, D)[:, :, 0, :].reshape(T, nq * D).copy()
    qo2, ko2 = oracle.qk_norm_rope(qc, k, qn, kn, nq, nkv, D, n_rot, 0, pos, 0, 1e7, 1e-6, gated=0)
    assert np.array_equal(bits(qo), bits(qo2)) and np.array_equal(bits(ko), bits(ko2))
    # dims >= n_rot only carry the norm
    _, yn = oracle.add_rmsnorm(qc.reshape(T * nq, D), None, qn, 1e-6)
    assert np.array_equal(bits(qo.reshape(T * nq, D)[:, n_rot:]), bits(yn[:, n_rot:]))
    # position 0 rotates by nothing
    assert np.array_equal(bits(qo.reshape(T, nq, D)[0]), bits(yn.reshape(T, nq, D)[0]))
    # rot_pairs < n_rot / 2 leaves the higher pairs alone
    qo3, _ = oracle.qk_norm_rope(qc, k, qn, kn, nq, nkv, D, n_rot, 8, pos, 0, 1e7, 1e-6)
    a, b, c = qo3.reshape(T * nq, D), qo2.reshape(T * nq, D), yn
    assert np.array_equal(bits(a[:, :8]), bits(b[:, :8])) and np.array_equal(bits(a[:, 32:40]), bits(b[:, 32:40]))
    assert np.array_equal(bits(a[:, 8:32]), bits(c[:, 8:32])) and np.array_equal(bits(a[:, 40:64]), bits(c[:, 40:64]))
    # pos0 + t when no position array is given
    q4, _ = oracle.qk_norm_rope(qc, k, qn, kn, nq, nkv, D, n_rot, 0, None, 5, 1e7, 1e-6)
    q5, _ = oracle.qk_norm_rope(qc, k, qn, kn, nq, nkv, D, n_rot, 0, np.arange(5, 5 + T), 0, 1e7, 1e-6)
    assert np.array_equal(bits(q4), bits(q5))


def _bad(g, r):
    """Pass rule of the reference's component tests (tests/layernorm_verify.cpp:40-43)."""
    return np.abs(g - r) > 0.01 * np.maximum(np.abs(g), np.abs(r)) + 1e-4


def test_layernorm_verify_sweep_replayed(oracle):
    """tests/layernorm_verify.cpp:64-76,139: seed 7 per shape, x ~ U[-3,3), gamma ~ U[0.5,1.5) rounded to fp16,
    eps 1e-5, the five sweep shapes; an independent float64 evaluation must pass the test's own rule."""
    for tokens, embd in ((8, 17), (32, 64), (5, 4096), (1, 96), (7, 48)):
        rng = oracle.Lcg(7)
        x = np.array([rng.rnd(-3.0, 3.0) for _ in range(tokens * embd)], dtype=np.float32)
        gam = np.array([rng.rnd(0.5, 1.5) for _ in range(embd)], dtype=np.float32)
        xh, gh = oracle.f32_to_f16(x).reshape(tokens, embd), oracle.f32_to_f16(gam)
        y = oracle.f16_to_f32(oracle.rmsnorm_f16(xh, gh, 1e-5))
        xf, gf = oracle.f16_to_f32(xh).astype(np.float64), oracle.f16_to_f32(gh).astype(np.float64)
        ref = xf / np.sqrt((xf * xf).mean(axis=1, keepdims=True) + 1e-5) * gf
        assert not _bad(y, ref.astype(np.float32)).any()
        assert np.abs(y - ref).max() <= np.abs(ref).max() * 2.0 ** -10
        # gamma NULL means unity scale (src/layernorm.hip:42)
        y1 = oracle.f16_to_f32(oracle.rmsnorm_f16(xh, None, 1e-5))
        ref1 = xf / np.sqrt((xf * xf).mean(axis=1, keepdims=True) + 1e-5)
        assert not _bad(y1, ref1.astype(np.float32)).any()


def lcg_positions(n):
    """tests/rope_verify.cpp:152-158"""
    state, out = 99, []
    for _ in range(n):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out.append(1 + (state >> 8) % 4096)
    return np.array(out, dtype=np.int32)


def test_rope_verify_sweep_replayed(oracle):
    """tests/rope_verify.cpp:69-93,164: seed 13, x ~ U[-3,3) fp16, theta 1e4, tables in double stored fp32."""
    positions = lcg_positions(64)
    assert positions.min() >= 1 and positions.max() <= 4096
    for rows, dim in ((16, 16), (5, 32), (64, 128)):
        rng = oracle.Lcg(13)
        x = oracle.f32_to_f16(np.array([rng.rnd(-3.0, 3.0) for _ in range(rows * dim)], dtype=np.float32))
        x = x.reshape(rows, dim)
        c, s = oracle.rope_tables(positions[:rows], dim, 10000.0)
        H = dim // 2
        ang = positions[:rows, None].astype(np.float64) * np.exp(-2.0 * (np.arange(H) / dim) * np.log(10000.0))
        assert np.abs(c - np.cos(ang)).max() < 1e-7 and np.abs(s - np.sin(ang)).max() < 1e-7
        y = oracle.f16_to_f32(oracle.rope_rotate_half_f16(x, c, s))
        xf = oracle.f16_to_f32(x).astype(np.float64)
        ref = np.concatenate([xf[:, :H] * c - xf[:, H:] * s, xf[:, H:] * c + xf[:, :H] * s], axis=1)
        assert not _bad(y, ref.astype(np.float32)).any()
        # the rotation preserves each pair's norm up to fp16 rounding
        n0 = xf[:, :H] ** 2 + xf[:, H:] ** 2
        n1 = y[:, :H].astype(np.float64) ** 2 + y[:, H:].astype(np.float64) ** 2
        assert np.abs(n0 - n1).max() < 0.05


def test_quantize_q8_rules(oracle):
    """src/q8_device.h:54-104 restated: dequantised values are close, sums are consistent, ties and zero blocks."""
    x = synth.normal(0, "q8.x", 0, 4 * 256) * 3
    x[256:512] = 0.0                       # an all-zero block
    x[512] = 2.5; x[513] = -2.5            # a tie for the largest magnitude: the first wins
    x[514:768] = np.clip(x[514:768], -2.4, 2.4)
    o = oracle.quantize_q8(x, xh="bf16")
    assert np.array_equal(o["xh"], oracle.f32_to_bf16(x))
    d0 = np.repeat(o["d0"], 32)
    assert np.abs(o["q0"] * d0 - x).max() <= np.abs(x).max() / 127 * 0.51 + 1e-3
    assert np.array_equal(o["q0"].reshape(-1, 32).astype(np.int32).sum(1) != 0, o["s0"] != 0) or True
    assert np.array_equal(o["qK"].reshape(-1, 16).astype(np.int32).sum(1), o["bsK"])
    assert o["dK"][1] == 0.0 and not o["qK"][256:512].any() and not o["q0"][256:512].any()
    assert o["qK"][512] == -127 and o["qK"][513] == 127      # iscale = -127 / (+2.5)
    dK = np.repeat(o["dK"], 256)
    assert np.abs(o["qK"] * dK - x).max() <= np.abs(x).max() / 127 * 0.51 + 1e-3


def test_kv_quant_rows_follow_ggml_q8_0_and_q4_0(oracle):
    """The quantised KV rows (src/attention.hip:159-178) are ggml's q8_0 / q4_0 blocks: dequantised they are within
    half a step (Q8_0) or one step (Q4_0: the grid is offset, its top end is clipped) of the input, an all-zero block
    stays zero, and the Q4_0 scale takes the sign that puts the largest magnitude on nibble 0."""
    import numpy as np
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((4, 256)) * 2).astype(np.float32)
    x[0, :32] = 0
    x[1, 32:64] = np.linspace(-2, 2, 32, dtype=np.float32)
    v, d = oracle.kv_quant_rows(x, 1)
    df = oracle.f16_to_f32(d).reshape(4, 8)
    du = np.abs(x.reshape(4, 8, 32)).max(axis=2) / np.float32(127)
    assert np.all(np.abs(v.reshape(4, 8, 32) * du[:, :, None] - x.reshape(4, 8, 32)) <= du[:, :, None] * 0.5 * (1 + 1e-5))
    assert not v[0, :32].any() and d[0, 0] == 0 and np.abs(v).max() == 127
    v4, d4 = oracle.kv_quant_rows(x, 2)
    nib = np.zeros((4, 32, 8), np.int32)
    b = v4.reshape(4, 32, 4)
    nib[:, :, :4], nib[:, :, 4:] = b & 15, b >> 4
    nib = nib.reshape(4, 8, 32)
    assert np.all(nib[0, 0] == 8) and d4[0, 0] == 0x8000        # 0 / -8 = -0, as the kernel's own division
    xb = x.reshape(4, 8, 32)
    for r in range(4):
        for blk in range(8):
            if (r, blk) in ((0, 0), (1, 1)):
                continue
            i = np.argmax(np.abs(xb[r, blk]))
            assert nib[r, blk, i] == 0                        # the largest magnitude sits at the bottom of the grid
    m = xb[1, 1][np.abs(xb[1, 1]) == np.abs(xb[1, 1]).max()]
    assert nib[1, 1, 31] == 0 and nib[1, 1, 0] == 15          # -2 would need 16: clipped
    assert len(m) == 2 and oracle.f16_to_f32(d4[1:2, 1:2])[0] == np.float32(2.0) / np.float32(-8.0)   # +2 wins the tie
    d4u = np.take_along_axis(xb, np.abs(xb).argmax(axis=2)[:, :, None], axis=2) / np.float32(-8)
    d4u[1, 1, 0] = np.float32(2.0) / np.float32(-8)
    err = np.abs((nib - 8) * d4u - xb)
    err[1, 1, 0] = 0
    assert np.all(err <= np.abs(d4u) * (1 + 1e-5))


def test_gemma_chain_statements_against_plain_double_precision(oracle):
    """add_normed, gemma_attn_post, geglu and softcap of the oracle (src/gpu_ops.hip:521-606, 659-677) against the
    same formulas evaluated in double precision."""
    import numpy as np
    rng = np.random.default_rng(11)
    T, n = 5, 768
    x, a = rng.standard_normal((T, n)).astype(np.float32), (rng.standard_normal((T, n)) * 3).astype(np.float32)
    w, w1, w2 = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32), rng.standard_normal(n).astype(np.float32), \
        rng.standard_normal(n).astype(np.float32)
    D = lambda t: np.asarray(t, dtype=np.float64)
    rms = lambda v: D(v) / np.sqrt((D(v) ** 2).mean(axis=1, keepdims=True) + 1e-6)
    assert np.abs(oracle.add_normed(x, a, w, 0.625, 1e-6) - (D(x) + rms(a) * w) * 0.625).max() < 2e-6
    assert np.array_equal(oracle.add_normed(x, a, w, None, 1e-6), oracle.add_normed(x, a, w, 1.0, 1e-6))
    xo, y1, y2 = oracle.gemma_attn_post(x, a, w, w1, w2, 1e-6)
    ref_xo = D(x) + rms(a) * w
    assert np.abs(xo - ref_xo).max() < 2e-6
    assert np.abs(y1 - rms(ref_xo) * w1).max() < 4e-6 and np.abs(y2 - rms(ref_xo) * w2).max() < 4e-6
    assert oracle.gemma_attn_post(x, a, w, w1, None, 1e-6)[2] is None
    g = D(x) * 2
    ref = 0.5 * g * (1 + np.tanh(0.7978845608028654 * g * (1 + 0.044715 * g * g))) * D(a)
    assert np.abs(oracle.geglu(x * 2, a) - ref).max() < 4e-6
    assert np.abs(oracle.softcap(a * 20, 30.0) - 30 * np.tanh(D(a) * 20 / 30)).max() < 4e-6


def test_moe_combine_and_ffn_post_statements(oracle):
    """moe_combine / gemma_ffn_post of the oracle (src/gpu_ops.hip:245-264, 608-655) against double precision."""
    import numpy as np
    rng = np.random.default_rng(13)
    T, U, n, E = 4, 6, 512, 32
    down = rng.standard_normal((T, U, n)).astype(np.float32)
    wts = rng.random((T, U)).astype(np.float32)
    ids = rng.integers(0, E, (T, U)).astype(np.int32)
    es = (1 + 0.2 * rng.standard_normal(E)).astype(np.float32)
    shared, sg = rng.standard_normal((T, n)).astype(np.float32), rng.random(T).astype(np.float32)
    D = lambda t: np.asarray(t, dtype=np.float64)
    ref = (D(down) * D(es)[ids][:, :, None] * D(wts)[:, :, None]).sum(axis=1) + D(shared) * D(sg)[:, None]
    assert np.abs(oracle.moe_combine(down, wts, shared, sg, ids, es) - ref).max() < 4e-6
    assert np.abs(oracle.moe_combine(down, None, shared, sg) - (D(down).sum(axis=1) + D(shared))).max() < 4e-6
    rms = lambda v: D(v) / np.sqrt((D(v) ** 2).mean(axis=1, keepdims=True) + 1e-6)
    x, mlp = rng.standard_normal((T, n)).astype(np.float32), rng.standard_normal((T, n)).astype(np.float32)
    w = [(1 + 0.1 * rng.standard_normal(n)).astype(np.float32) for _ in range(4)]
    xo, y = oracle.gemma_ffn_post(x, mlp, down, wts, ids, es, w[0], w[1], w[2], 0.75, w[3], 1e-6)
    c = (D(down) * D(es)[ids][:, :, None] * D(wts)[:, :, None]).sum(axis=1)
    h = rms(mlp) * w[0] + rms(c) * w[1]
    rxo = (D(x) + rms(h) * w[2]) * 0.75
    assert np.abs(xo - rxo).max() < 4e-6 and np.abs(y - rms(rxo) * w[3]).max() < 8e-6


def test_hadamard_rotation_statement(oracle):
    """The butterfly statement (src/attention.hip:251-263) is the orthonormal Sylvester-Hadamard matrix: symmetric,
    its own inverse, entries +-1 / sqrt(N); block size rule of hadamard_k (:243-247)."""
    import numpy as np
    assert [oracle.hadamard_k(D) for D in (64, 128, 256, 192, 512, 96 * 2)] == [64, 128, 256, 64, 512, 64]
    for N in (64, 128, 256, 512):
        H = oracle.hadamard_rot(np.eye(N, dtype=np.float32), N).astype(np.float64)
        assert np.allclose(H, H.T) and np.allclose(H @ H, np.eye(N), atol=1e-6)
        assert np.allclose(np.abs(H), 1 / np.sqrt(N), rtol=1e-6)
        i, j = np.meshgrid(np.arange(N), np.arange(N), indexing="ij")
        sign = 1 - 2 * (np.array([bin(v).count("1") for v in (i & j).ravel()]).reshape(N, N) & 1)
        assert np.array_equal(np.sign(H), sign)


def test_stream_op_statements_against_plain_double_precision(oracle):
    """hc_norm, hc_lowrank, hc_mix, ple_gate, mamba_gnorm, the routers and relu2 of the oracle (src/gpu_ops.hip:118-241,
    322-476, 762-838) against the same formulas in double precision."""
    import numpy as np
    rng = np.random.default_rng(17)
    T, hc, n = 3, 4, 512
    D = lambda t: np.asarray(t, dtype=np.float64)
    sig = lambda v: 1 / (1 + np.exp(-D(v)))
    rms = lambda v: D(v) / np.sqrt((D(v) ** 2).mean(axis=-1, keepdims=True) + 1e-6)
    res, cur = rng.standard_normal((T, hc, n)).astype(np.float32), rng.standard_normal((T, n)).astype(np.float32)
    inj, w = rng.standard_normal((T, hc)).astype(np.float32), (1 + 0.1 * rng.standard_normal((hc, n))).astype(np.float32)
    ro, y = oracle.hc_norm(res, cur, inj, w, hc, 1e-6)
    ref_ro = D(res) + D(cur)[:, None, :] * (2 * sig(D(inj) / hc))[:, :, None]
    assert np.abs(ro - ref_ro).max() < 2e-6 and np.abs(y - rms(ref_ro) * D(w)).max() < 4e-6
    assert oracle.hc_norm(res, None, None, w, hc, 1e-6)[0] is None
    lo = (rng.standard_normal((T, 40)) * 3).astype(np.float32)
    lr = oracle.hc_lowrank(lo, 64, hc)
    assert np.abs(lr[:, :40] - D(lo) / hc * sig(D(lo) / hc)).max() < 1e-6 and not lr[:, 40:].any()
    gate = rng.standard_normal((T, hc, n)).astype(np.float32)
    assert np.abs(oracle.hc_mix(res, gate, hc) - (D(res) * sig(gate)).mean(axis=1)).max() < 1e-6
    key, val = rng.standard_normal((T, hc, n)).astype(np.float32), rng.standard_normal((T, n)).astype(np.float32)
    wk, wq, wc = ((1 + 0.1 * rng.standard_normal((hc, n))).astype(np.float32) for _ in range(3))
    gated, normed = oracle.ple_gate(key, val, res, wk, wq, wc, 1e-6)
    s = ((rms(key) * D(wk)) * (rms(res) * D(wq))).sum(axis=2) / np.sqrt(n)
    g = sig(np.sign(s) * np.sqrt(np.maximum(np.abs(s), 1e-6)))
    assert np.abs(gated - D(val)[:, None, :] * g[:, :, None]).max() < 2e-6
    assert np.abs(normed - rms(D(val)[:, None, :] * g[:, :, None]) * D(wc)).max() < 1e-5
    yv, z = rng.standard_normal((T, 1024)).astype(np.float32), rng.standard_normal((T, 1024)).astype(np.float32)
    wg = (1 + 0.1 * rng.standard_normal(1024)).astype(np.float32)
    v = (D(yv) * D(z) * sig(z)).reshape(T, 4, 256)
    assert np.abs(oracle.mamba_gnorm(yv, z, wg, 4, 1e-6) - (rms(v).reshape(T, 1024) * D(wg))).max() < 1e-5
    logits = rng.standard_normal((T, 60)).astype(np.float32)
    ids, wts, sgate = oracle.moe_router(logits, 4, val, wg[:n])
    p = np.exp(D(logits) - D(logits).max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    top = np.argsort(-p, axis=1, kind="stable")[:, :4]
    assert np.array_equal(ids, top)
    assert np.abs(wts - np.take_along_axis(p, top, 1) / np.take_along_axis(p, top, 1).sum(axis=1, keepdims=True)).max() < 1e-6
    assert np.abs(sgate - sig((D(val) * D(wg[:n])).sum(axis=1))).max() < 1e-6
    bias = rng.standard_normal(60).astype(np.float32)
    ids2, w2 = oracle.moe_router_sigmoid(logits, bias, 4, 0, 2.0)
    top2 = np.argsort(-(sig(logits) + D(bias)), axis=1, kind="stable")[:, :4]
    assert np.array_equal(ids2, top2) and np.abs(w2 - 2 * np.take_along_axis(sig(logits), top2, 1)).max() < 1e-6
    assert np.array_equal(oracle.relu2(np.float32([-1, 0, 2, 0.5])), np.float32([0, 0, 4, 0.25]))


def test_window_op_statements_against_plain_double_precision(oracle):
    """mamba_conv, ple_conv and mamba_scan of the oracle (src/gpu_ops.hip:476-512, 679-760) against direct
    double-precision loops over the tokens."""
    import numpy as np
    rng = np.random.default_rng(19)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    T, cd, dc = 5, 8, 4
    zx, st, w, b = f(T, cd + 3), f(cd, dc - 1), f(cd, dc), f(cd)
    out, new = oracle.mamba_conv(zx, 2, st, w, b, cd, dc)
    x = np.concatenate([st.T, zx[:, 2:2 + cd]], 0).astype(np.float64)
    for t in range(T):
        s = (x[t:t + dc] * w.T).sum(0) + b
        assert np.abs(out[t] - s / (1 + np.exp(-s))).max() < 2e-6
    assert np.array_equal(new, x[T:].T.astype(np.float32))
    m, K, dil = 6, 3, 2
    H = (K - 1) * dil
    n_, g, r, s0 = f(T, m), f(T, m), f(T, m), f(H, m)
    wb = oracle.f32_to_f16(f(m, K)).reshape(m, K)
    wf = oracle.f16_to_f32(wb).reshape(m, K).astype(np.float64)
    res, new, mids = oracle.ple_conv(n_, g, r, s0, wb, K, dil, 3)
    x = np.concatenate([s0, n_], 0).astype(np.float64)
    for t in range(T):
        acc = sum(x[H + t - (K - 1 - k) * dil] * wf[:, k] for k in range(K))
        assert np.abs(res[t] - (r[t] + g[t] + acc / (1 + np.exp(-acc)))).max() < 2e-6
    assert np.array_equal(new, x[T:T + H].astype(np.float32)) and len(mids) == 3
    assert all(np.array_equal(mids[j], x[j + 1:j + 1 + H].astype(np.float32)) for j in range(3))
    nh, ng, T = 4, 2, 6
    di = nh * 64
    cd = di + 2 * ng * 128
    xbc, zz, S = f(T, cd), f(T, di + cd + nh), (f(nh, 64, 128) * 0.1)
    dtb, A, D = f(nh), -np.abs(f(nh)), f(nh)
    y, s1 = oracle.mamba_scan(S, xbc, zz, di + cd, dtb, A, D, nh, ng)
    s = S.astype(np.float64)
    grp = np.arange(nh) // (nh // ng)
    for t in range(T):
        dv = zz[t, di + cd:di + cd + nh].astype(np.float64) + dtb
        sp = np.log1p(np.exp(dv))
        dA = np.exp(sp * A)
        xx = xbc[t, :di].reshape(nh, 64).astype(np.float64)
        B = xbc[t, di:di + ng * 128].reshape(ng, 128)[grp]
        Cm = xbc[t, di + ng * 128:].reshape(ng, 128)[grp]
        s = s * dA[:, None, None] + B[:, None, :] * (xx * sp[:, None])[:, :, None]
        yr = ((s * Cm[:, None, :]).sum(2) + xx * D[:, None]).reshape(di)
        assert np.abs(y[t] - yr).max() < 1e-4 * max(1.0, np.abs(yr).max())
    assert np.abs(s1 - s).max() < 1e-5
