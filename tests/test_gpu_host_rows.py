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
