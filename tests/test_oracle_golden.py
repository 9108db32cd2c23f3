"""The CPU restatement (oracle/oracle_ops.c) against golden vectors made by the reference's own CPU functions
(tests/golden/make_golden.py) and, where the reference build is present, against that build directly. Bit-exact."""
import ctypes as C
import os

import numpy as np
import pytest

from rocm_hip_b200 import synth

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(G, name))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_rmsnorm_golden(oracle):
    g = load("rmsnorm.npz")
    for name in ("h1024", "d128", "n17", "n5120"):
        x, want = g[name + "_x"], g[name + "_y"]
        w = g[name + "_w"] if name + "_w" in g else None
        _, y = oracle.add_rmsnorm(x, None, w, float(g[name + "_eps"]))
        assert np.array_equal(bits(y), bits(want)), name


def test_rope_neox_golden(oracle):
    g = load("rope_neox.npz")
    pos = g["positions"]
    for name, D, n_rot, base in (("d128_full_1e6", 128, 128, 1e6), ("d256_rot64_1e7", 256, 64, 1e7),
                                  ("d64_full_1e4", 64, 64, 1e4)):
        x, want = g[name + "_x"], g[name + "_y"]
        out = x.copy()
        for r, p in enumerate(pos):
            oracle.port().orc_rope_neox(oracle.ptr(out[r]), n_rot, int(p), base)
        assert np.array_equal(bits(out), bits(want)), name
        # the extended form with all pairs rotating and no frequency factors is the same function
        out2 = x.copy()
        for r, p in enumerate(pos):
            oracle.port().orc_rope_neox_ex(oracle.ptr(out2[r]), n_rot, 0, int(p), base, None)
        assert np.array_equal(bits(out2), bits(want)), name
        # and so is the head-level q/k path without the norm (one head per token, per-row positions)
        q, _ = oracle.qk_norm_rope(x, None, None, None, 1, 0, D, n_rot, 0, pos, 0, base, 1e-6, do_norm=0)
        assert np.array_equal(bits(q), bits(want)), name


def test_silu_golden(oracle):
    g = load("silu.npz")
    got = np.array([oracle.port().orc_silu(float(v)) for v in g["g"]], dtype=np.float32)
    assert np.array_equal(bits(got), bits(g["silu"]))
    u = synth.normal(1, "silu.u", 0, g["g"].size)
    with np.errstate(over="ignore", invalid="ignore"):
        assert np.array_equal(bits(oracle.swiglu(g["g"], u)), bits(g["silu"] * u))


def test_dequant_golden(oracle):
    g = load("dequant.npz")
    for name, qt in (("q8_0", oracle.Q8_0), ("q4_0", oracle.Q4_0)):
        tab, want = g[name + "_table"], g[name + "_out"]
        rows, E = want.shape
        assert oracle.port().orc_row_size(qt, E) == tab.shape[1]
        st, out = oracle.embed_rows(qt, tab, tab.shape[1], rows, np.arange(rows), E)
        assert st == 0 and np.array_equal(bits(out), bits(want)), name
        # a permuted gather returns the permuted rows
        perm = synth.randint(3, "perm", 0, 200, 0, rows)
        st, out = oracle.embed_rows(qt, tab, tab.shape[1], rows, perm, E)
        assert st == 0 and np.array_equal(bits(out), bits(want[perm])), name
        # the id range check of the gather loop
        for bad in (-1, rows):
            st, _ = oracle.embed_rows(qt, tab, tab.shape[1], rows, np.array([0, bad, 1]), E)
            assert st == -1
    assert oracle.port().orc_row_size(oracle.Q8_0, 33) == 0
    assert oracle.port().orc_to_float(9, None, None, 32) == -1        # (ggml id 9, Q8_1, is not a row format here)


def test_dequant_golden_other_row_formats(oracle):
    """F32 / F16 / BF16 / Q4_1 / Q5_0 / Q5_1 / Q4_K / Q5_K / Q6_K rows: the restatement against the reference build's
    qt_to_float on random payloads (every bit pattern of the packed fields occurs), finite scales of both signs and the
    special fp16 scales (zero, subnormal, largest, negative), bit for bit."""
    g = load("dequant_more.npz")
    for qt in (oracle.F32, oracle.F16, oracle.BF16, oracle.Q4_1, oracle.Q5_0, oracle.Q5_1, oracle.Q4_K, oracle.Q5_K,
               oracle.Q6_K):
        tab, want = g["t%d_table" % qt], g["t%d_out" % qt]
        rows, E = want.shape
        blk, bb = oracle.BLOCK[qt]
        assert oracle.port().orc_row_size(qt, E) == tab.shape[1] == E // blk * bb
        assert oracle.port().orc_row_size(qt, E + 1) == (0 if blk > 1 else (E + 1) * bb)
        st, out = oracle.embed_rows(qt, tab, tab.shape[1], rows, np.arange(rows), E)
        assert st == 0
        ok = ~np.isnan(want)                                   # (a NaN scale has no defined payload)
        assert np.array_equal(bits(out)[ok], bits(want)[ok]) and np.array_equal(np.isnan(out), np.isnan(want)), qt
        perm = synth.randint(3, "perm2", 0, 50, 0, rows)
        st, out = oracle.embed_rows(qt, tab, tab.shape[1], rows, perm, E, scale=0.125)
        assert st == 0 and np.array_equal(bits(out)[ok[perm]], bits((want[perm] * np.float32(0.125)).astype(np.float32))[ok[perm]])


def test_half_tables_golden(oracle):
    g = load("half_tables.npz")
    h = np.arange(65536, dtype=np.uint32)
    got = np.array([oracle.port().orc_fp16_to_fp32(int(v)) for v in h], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), g["fp16_bits"])
    # (signalling NaN payloads are quieted on their way through a float return value: compare the rest)
    b = oracle.bf16_to_f32(h.astype(np.uint16))
    okb = ~np.isnan(b)
    assert np.array_equal(b.view(np.uint32)[okb], g["bf16_bits"][okb]) and okb.sum() == 65536 - 2 * 127
    # numpy's fp16 widening (used to build test inputs) agrees with the reference's on every non-NaN pattern
    f = oracle.f16_to_f32(h.astype(np.uint16))
    ok = ~np.isnan(f)
    assert np.array_equal(f.view(np.uint32)[ok], g["fp16_bits"][ok])


def test_narrowing_conversions(oracle):
    x = np.concatenate([synth.normal(0, "cvt", 0, 20000) * 50, np.array(
        [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5, 6.0975552e-5, np.inf,
         -np.inf], dtype=np.float32)])
    got = np.array([oracle.port().orc_fp32_to_fp16(float(v)) for v in x], dtype=np.uint16)
    with np.errstate(over="ignore"):
        assert np.array_equal(got, oracle.f32_to_f16(x))
    gotb = np.array([oracle.port().orc_fp32_to_bf16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(gotb, oracle.f32_to_bf16(x))
    # round to nearest even on a tie and just off it
    for u, want in ((0x3F808000, 0x3F80), (0x3F818000, 0x3F82), (0x3F808001, 0x3F81), (0x3F807FFF, 0x3F80)):
        f = np.array([u], dtype=np.uint32).view(np.float32)[0]
        assert oracle.port().orc_fp32_to_bf16(float(f)) == want


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(G), "..", "oracle", "_ref", "libref_cpu.so")),
                    reason="reference build (oracle/_ref) not present")
def test_runner_port_equals_reference(oracle):
    """The row-parallel runner gives the same bits with the restatement and with the reference's functions, on the
    Qwen3-0.6B shapes at a reduced token count, for 1 and several threads."""
    P, R = oracle.port(), oracle.ref()
    assert R.cpu_is_reference() == 1 and P.cpu_is_reference() == 0
    p = oracle.ptr
    T, E, FF, nq, nkv, D = 37, 1024, 3072, 16, 8, 128
    x = synth.normal(0, "rp.x", 0, T * E).reshape(T, E)
    a = synth.normal(0, "rp.a", 0, T * E).reshape(T, E)
    w = synth.normal(0, "rp.w", 0, E, 1.0, 0.1)
    outs = []
    for lib, nth in ((P, 1), (R, 1), (R, 3)):
        xo, y = np.empty_like(x), np.empty_like(x)
        lib.cpu_add_rmsnorm(p(x), p(a), p(xo), p(w), p(y), E, T, 1e-6, nth)
        outs.append((xo, y))
    for xo, y in outs[1:]:
        assert np.array_equal(bits(xo), bits(outs[0][0])) and np.array_equal(bits(y), bits(outs[0][1]))

    g = synth.normal(0, "rp.g", 0, T * FF)
    u = synth.normal(0, "rp.u", 0, T * FF)
    o1, o2 = np.empty_like(g), np.empty_like(g)
    P.cpu_swiglu(p(g), p(u), p(o1), g.size, 2)
    R.cpu_swiglu(p(g), p(u), p(o2), g.size, 3)
    assert np.array_equal(bits(o1), bits(o2)) and np.array_equal(bits(o1), bits(oracle.swiglu(g, u)))

    q = synth.normal(0, "rp.q", 0, T * nq * D).reshape(T, nq * D)
    k = synth.normal(0, "rp.k", 0, T * nkv * D).reshape(T, nkv * D)
    qn, kn = synth.normal(0, "rp.qn", 0, D, 1.0, 0.1), synth.normal(0, "rp.kn", 0, D, 1.0, 0.1)
    pos = synth.randint(0, "rp.pos", 0, T, 0, 32768).astype(np.int32)
    res = []
    for lib, nth in ((P, 1), (R, 2)):
        qo, ko = np.empty_like(q), np.empty_like(k)
        lib.cpu_qk_norm_rope(p(q), p(k), p(qn), p(kn), p(qo), p(ko), nq, nkv, D, D, p(pos), 0, T, 1e6, 1e-6, 0, 1, nth)
        res.append((qo, ko))
    assert np.array_equal(bits(res[0][0]), bits(res[1][0])) and np.array_equal(bits(res[0][1]), bits(res[1][1]))
    qo, ko = oracle.qk_norm_rope(q, k, qn, kn, nq, nkv, D, D, 0, pos, 0, 1e6, 1e-6)
    assert np.array_equal(bits(qo), bits(res[1][0])) and np.array_equal(bits(ko), bits(res[1][1]))

    vocab = 500
    for qt, maker in ((oracle.Q8_0, synth.q8_0_table), (oracle.Q4_0, synth.q4_0_table)):
        tab = maker(0, "rp.tab", vocab, E)
        ids = synth.randint(0, "rp.ids", 0, T, 0, vocab).astype(np.int32)
        e1, e2 = np.empty((T, E), np.float32), np.empty((T, E), np.float32)
        assert P.cpu_embed_rows(qt, p(tab), tab.shape[1], vocab, p(ids), p(e1), E, T, 1.0, 1) == 0
        assert R.cpu_embed_rows(qt, p(tab), tab.shape[1], vocab, p(ids), p(e2), E, T, 1.0, 4) == 0
        assert np.array_equal(bits(e1), bits(e2))
        ids[5] = vocab
        assert R.cpu_embed_rows(qt, p(tab), tab.shape[1], vocab, p(ids), p(e2), E, T, 1.0, 2) == -1
