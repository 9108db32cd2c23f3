"""The host-buffer entry points (b200_host_*): rows in host memory streamed through the device in chunks give exactly
the bits of the device launchers on the same rows, whatever the chunking, and agree with the CPU oracle."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import bf16_ulp_dist, dev, host, max_rel_rows

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hr(ops):
    h = ops.HostRows(slot_bytes=1 << 20, n_slots=3)   # small slots: many chunks, ragged last chunk
    yield h
    h.close()


def test_add_rmsnorm_and_swiglu(ops, oracle, hr):
    T, n = 1237, 1024
    for bf16 in (False, True):
        x = synth.normal(0, "h.x", 0, T * n).reshape(T, n)
        a = synth.normal(0, "h.a", 0, T * n).reshape(T, n)
        w = synth.normal(0, "h.w", 0, n, 1.0, 0.1)
        if bf16:
            x, a = oracle.f32_to_bf16(x).reshape(T, n), oracle.f32_to_bf16(a).reshape(T, n)
        xo, y = np.zeros_like(x), np.zeros_like(x)
        hr.add_rmsnorm(x, a, xo, w, y, n, T, 1e-6)
        dt = torch.bfloat16 if bf16 else None
        dxo, dy = torch.zeros_like(dev(x, dt)), torch.zeros_like(dev(x, dt))
        ops.gpu_add_rmsnorm(dev(x, dt), dev(a, dt), dxo, dev(w), dy, n, T, 1e-6)
        torch.cuda.synchronize()
        assert np.array_equal(xo, host(dxo)) and np.array_equal(y.view(np.uint8), host(dy).view(np.uint8))
        y2 = np.zeros_like(x)
        hr.add_rmsnorm(x, None, None, w, y2, n, T, 1e-6)
        if bf16:
            assert bf16_ulp_dist(y2, oracle.add_rmsnorm_bf16(x, None, w, 1e-6)[1]).max() <= 1
        else:
            assert max_rel_rows(y2, oracle.add_rmsnorm(x, None, w, 1e-6)[1]) <= 1e-5
    rows, width = 999, 3072
    g, u = synth.normal(0, "h.g", 0, rows * width), synth.normal(0, "h.u", 0, rows * width)
    out = np.zeros_like(g)
    hr.swiglu(g, u, out, rows, width)
    assert max_rel_rows(out.reshape(rows, width), oracle.swiglu(g, u).reshape(rows, width)) <= 1e-5


def test_qk_norm_rope_positions_follow_chunks(ops, oracle, hr):
    """pos0 + t must mean the row's global index, not its index inside a chunk."""
    T, nq, nkv, D = 700, 16, 8, 128
    q = synth.normal(0, "h.q", 0, T * nq * D).reshape(T, nq * D)
    k = synth.normal(0, "h.k", 0, T * nkv * D).reshape(T, nkv * D)
    qn, kn = synth.normal(0, "h.qn", 0, D, 1.0, 0.1), synth.normal(0, "h.kn", 0, D, 1.0, 0.1)
    qo, ko = np.zeros_like(q), np.zeros_like(k)
    hr.qk_norm_rope(q, k, qn, kn, qo, ko, nq, nkv, D, D, 0, None, 1000, T, 1e6, 1e-6)
    wq, wk = oracle.qk_norm_rope(q, k, qn, kn, nq, nkv, D, D, 0, None, 1000, 1e6, 1e-6)
    assert max_rel_rows(qo.reshape(-1, D), wq.reshape(-1, D)) <= 1e-5 and max_rel_rows(ko.reshape(-1, D), wk.reshape(-1, D)) <= 1e-5
    pos = synth.randint(0, "h.pos", 0, T, 0, 32768).astype(np.int32)
    qb, kb = oracle.f32_to_bf16(q).reshape(q.shape), oracle.f32_to_bf16(k).reshape(k.shape)
    qo, ko = np.zeros_like(qb), np.zeros_like(kb)
    hr.qk_norm_rope(qb, kb, qn, kn, qo, ko, nq, nkv, D, D, 0, pos, 0, T, 1e6, 1e-6)
    wq, wk = oracle.qk_norm_rope(qb, kb, qn, kn, nq, nkv, D, D, 0, pos, 0, 1e6, 1e-6, bf16=True)
    assert bf16_ulp_dist(qo, wq).max() <= 1 and bf16_ulp_dist(ko, wk).max() <= 1


def test_embed_rows(ops, oracle, hr):
    vocab, E, T = 3000, 1024, 2427
    table = synth.q8_0_table(0, "h.tab", vocab, E)
    ids = synth.randint(0, "h.ids", 0, T, 0, vocab).astype(np.int32)
    out = np.zeros((T, E), np.float32)
    dt = dev(table)
    hr.embed_rows(ops.QT_Q8_0, dt, table.shape[1], vocab, ids, out, E, T)
    _, want = oracle.embed_rows(oracle.Q8_0, table, table.shape[1], vocab, ids, E)
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    ids[1234] = vocab
    with pytest.raises(ops.LayerOpError) as e:
        hr.embed_rows(ops.QT_Q8_0, dt, table.shape[1], vocab, ids, out, E, T)
    assert e.value.code == 1


def test_row_too_large_for_a_slot(ops, hr):
    x = np.zeros((2, 1 << 19), np.float32)     # 2 MB per row, slots are 1 MB
    with pytest.raises(ops.LayerOpError) as e:
        hr.add_rmsnorm(x, None, None, None, x.copy(), 1 << 19, 2, 1e-6)
    assert e.value.code == 1


@pytest.mark.parametrize("bf16", [False, True])
def test_layer_sweep_gives_the_bits_of_the_six_calls(ops, oracle, bf16):
    """b200_host_layer_sweep keeps the residual stream on the device between the kernels of a chunk; every output
    row must still be, bit for bit, what the six separate host-buffer calls produce (and the gather the oracle's)."""
    T, E, nq, nkv, D, FF, vocab = 333, 1024, 16, 8, 128, 3072, 2000
    h = ops.HostRows(slot_bytes=4 << 20, n_slots=3)    # 17 rows per chunk: many chunks, a ragged last one
    try:
        f = lambda name, *shape: synth.normal(5, name, 0, int(np.prod(shape))).reshape(shape)
        cv = (lambda a: oracle.f32_to_bf16(a).reshape(a.shape)) if bf16 else (lambda a: a)
        table = synth.q8_0_table(0, "ls.tab", vocab, E)
        ids = synth.randint(0, "ls.ids", 0, T, 0, vocab).astype(np.int32)
        q, k = cv(f("ls.q", T, nq * D)), cv(f("ls.k", T, nkv * D))
        p1, p2, g, u = cv(f("ls.p1", T, E)), cv(f("ls.p2", T, E)), cv(f("ls.g", T, FF)), cv(f("ls.u", T, FF))
        w1, w2, w3 = (synth.normal(5, n, 0, E, 1.0, 0.1) for n in ("ls.w1", "ls.w2", "ls.w3"))
        qn, kn = synth.normal(5, "ls.qn", 0, D, 1.0, 0.1), synth.normal(5, "ls.kn", 0, D, 1.0, 0.1)
        z = lambda *shape: np.zeros(shape, q.dtype)
        dt = dev(table)
        # the six calls
        x, xn1, qo, ko, xa, xn2, act, x3, xn3 = z(T, E), z(T, E), z(T, nq * D), z(T, nkv * D), z(T, E), z(T, E), z(T, FF), z(T, E), z(T, E)
        h.embed_rows(ops.QT_Q8_0, dt, table.shape[1], vocab, ids, x, E, T)
        h.add_rmsnorm(x, None, None, w1, xn1, E, T, 1e-6)
        h.qk_norm_rope(q, k, qn, kn, qo, ko, nq, nkv, D, D, 0, None, 77, T, 1e6, 1e-6)
        h.add_rmsnorm(x, p1, xa, w2, xn2, E, T, 1e-6)
        h.swiglu(g, u, act, T, FF)
        h.add_rmsnorm(xa, p2, x3, w3, xn3, E, T, 1e-6)
        # one call
        s_xn1, s_qo, s_ko, s_xn2, s_act, s_x3, s_xn3 = z(T, E), z(T, nq * D), z(T, nkv * D), z(T, E), z(T, FF), z(T, E), z(T, E)
        h.layer_sweep(qtype=ops.QT_Q8_0, table_dev=dt, row_bytes=table.shape[1], vocab=vocab, tokens=ids, E=E,
                      w_attn_norm=w1, w_ffn_norm=w2, w_next_norm=w3, eps=1e-6, xn_attn=s_xn1, qfull=q, k=k, q_out=s_qo,
                      k_out=s_ko, q_norm=qn, k_norm=kn, n_q=nq, n_kv=nkv, head_dim=D, n_rot=D, freq_base=1e6,
                      attn_proj=p1, xn_ffn=s_xn2, gate=g, up=u, FF=FF, act=s_act, ffn_proj=p2, x_out=s_x3, xn_next=s_xn3,
                      T=T, pos0=77)
        for a, b in ((xn1, s_xn1), (qo, s_qo), (ko, s_ko), (xn2, s_xn2), (act, s_act), (x3, s_x3), (xn3, s_xn3)):
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
        if not bf16:   # and the chain is the oracle's: gather bit-exact, hence x3 = (embed + p1) + p2 exactly
            _, want = oracle.embed_rows(oracle.Q8_0, table, table.shape[1], vocab, ids, E)
            assert np.array_equal(s_x3, (want + p1) + p2)
        ids[7] = -1
        with pytest.raises(ops.LayerOpError) as e:
            h.layer_sweep(qtype=ops.QT_Q8_0, table_dev=dt, row_bytes=table.shape[1], vocab=vocab, tokens=ids, E=E,
                          w_attn_norm=w1, w_ffn_norm=w2, w_next_norm=w3, eps=1e-6, xn_attn=s_xn1, qfull=q, k=k,
                          q_out=s_qo, k_out=s_ko, q_norm=qn, k_norm=kn, n_q=nq, n_kv=nkv, head_dim=D, n_rot=D,
                          freq_base=1e6, attn_proj=p1, xn_ffn=s_xn2, gate=g, up=u, FF=FF, act=s_act, ffn_proj=p2,
                          x_out=s_x3, xn_next=s_xn3, T=T, pos0=77)
        assert e.value.code == 1
    finally:
        h.close()
