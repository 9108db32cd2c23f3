"""Row sharding over several GPUs from one process (b200_host_group_*): whatever the number of devices, every row gets
the bits the single-device host-buffer context gives it. Runs with one device too (a group of one); the wider groups
are exercised on a box that has more."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth

pytestmark = pytest.mark.gpu


def _sizes():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 1
    return sorted({1, min(2, n), n})


@pytest.fixture(scope="module")
def single(ops):
    h = ops.HostRows(slot_bytes=1 << 20, n_slots=3)
    yield h
    h.close()


@pytest.mark.parametrize("G", _sizes())
def test_group_equals_single_device(ops, single, G):
    grp = ops.HostGroup(G, slot_bytes=1 << 20, n_slots=3)
    try:
        assert grp.size == G
        T, n = 1013, 1024                                  # not a multiple of any group size
        x = synth.normal(0, "g.x", 0, T * n).reshape(T, n)
        a = synth.normal(0, "g.a", 0, T * n).reshape(T, n)
        w = synth.normal(0, "g.w", 0, n, 1.0, 0.1)
        got = [np.zeros_like(x) for _ in range(2)]
        want = [np.zeros_like(x) for _ in range(2)]
        grp.add_rmsnorm(x, a, got[0], w, got[1], n, T, 1e-6)
        single.add_rmsnorm(x, a, want[0], w, want[1], n, T, 1e-6)
        assert all(np.array_equal(g.view(np.uint32), s.view(np.uint32)) for g, s in zip(got, want))

        rows, width = 777, 3072
        g_, u_ = synth.normal(0, "g.g", 0, rows * width), synth.normal(0, "g.u", 0, rows * width)
        o1, o2 = np.zeros_like(g_), np.zeros_like(g_)
        grp.swiglu(g_, u_, o1, rows, width)
        single.swiglu(g_, u_, o2, rows, width)
        assert np.array_equal(o1.view(np.uint32), o2.view(np.uint32))

        # positions: explicit, and pos0 + global row index across the device ranges
        Tq, nq, nkv, D = 701, 16, 8, 128
        q = synth.normal(0, "g.q", 0, Tq * nq * D).reshape(Tq, nq * D)
        k = synth.normal(0, "g.k", 0, Tq * nkv * D).reshape(Tq, nkv * D)
        qn, kn = synth.normal(0, "g.qn", 0, D, 1.0, 0.1), synth.normal(0, "g.kn", 0, D, 1.0, 0.1)
        pos = synth.randint(0, "g.pos", 0, Tq, 0, 32768).astype(np.int32)
        for p, p0 in ((None, 1000), (pos, 0)):
            qa, ka, qb, kb = np.zeros_like(q), np.zeros_like(k), np.zeros_like(q), np.zeros_like(k)
            grp.qk_norm_rope(q, k, qn, kn, qa, ka, nq, nkv, D, D, 0, p, p0, Tq, 1e6, 1e-6)
            single.qk_norm_rope(q, k, qn, kn, qb, kb, nq, nkv, D, D, 0, p, p0, Tq, 1e6, 1e-6)
            assert np.array_equal(qa.view(np.uint32), qb.view(np.uint32))
            assert np.array_equal(ka.view(np.uint32), kb.view(np.uint32))

        vocab, E, Te = 3000, 1024, 2427
        table = synth.q8_0_table(0, "g.tab", vocab, E)
        ids = synth.randint(0, "g.ids", 0, Te, 0, vocab).astype(np.int32)
        tabs = [torch.from_numpy(table).to(f"cuda:{d}") for d in range(G)]
        e1, e2 = np.zeros((Te, E), np.float32), np.zeros((Te, E), np.float32)
        grp.embed_rows(ops.QT_Q8_0, tabs, table.shape[1], vocab, ids, e1, E, Te)
        single.embed_rows(ops.QT_Q8_0, tabs[0], table.shape[1], vocab, ids, e2, E, Te)
        assert np.array_equal(e1.view(np.uint32), e2.view(np.uint32))
        ids[Te - 1] = -1                                   # a bad id in the last device's range: refused up front
        before = e1.copy()
        with pytest.raises(ops.LayerOpError) as err:
            grp.embed_rows(ops.QT_Q8_0, tabs, table.shape[1], vocab, ids, e1, E, Te)
        assert err.value.code == 1 and np.array_equal(e1, before)
        ids[Te - 1] = 5

        # the whole layer sweep: rows, positions (pos0 + the global row) and the per-device tables follow the ranges
        Ts, FF = 517, 1536
        f = lambda name, *shape: synth.normal(3, name, 0, int(np.prod(shape))).reshape(shape)
        qs, ks, p1, p2, gs, us = f("s.q", Ts, nq * D), f("s.k", Ts, nkv * D), f("s.p1", Ts, E), f("s.p2", Ts, E), f("s.g", Ts, FF), f("s.u", Ts, FF)
        w1, w2, w3 = (synth.normal(3, n_, 0, E, 1.0, 0.1) for n_ in ("s.w1", "s.w2", "s.w3"))
        outs = []
        for runner, tab_kw in ((grp, dict(tables_dev=tabs)), (single, dict(table_dev=tabs[0]))):
            o = [np.zeros((Ts, E), np.float32), np.zeros((Ts, nq * D), np.float32), np.zeros((Ts, nkv * D), np.float32),
                 np.zeros((Ts, E), np.float32), np.zeros((Ts, FF), np.float32), np.zeros((Ts, E), np.float32), np.zeros((Ts, E), np.float32)]
            runner.layer_sweep(qtype=ops.QT_Q8_0, row_bytes=table.shape[1], vocab=vocab, tokens=ids[:Ts], E=E, w_attn_norm=w1,
                               w_ffn_norm=w2, w_next_norm=w3, eps=1e-6, xn_attn=o[0], qfull=qs, k=ks, q_out=o[1], k_out=o[2],
                               q_norm=qn, k_norm=kn, n_q=nq, n_kv=nkv, head_dim=D, n_rot=D, freq_base=1e6, attn_proj=p1,
                               xn_ffn=o[3], gate=gs, up=us, FF=FF, act=o[4], ffn_proj=p2, x_out=o[5], xn_next=o[6], T=Ts,
                               pos0=123, **tab_kw)
            outs.append(o)
        for a_, b_ in zip(*outs):
            assert a_.any() and np.array_equal(a_.view(np.uint32), b_.view(np.uint32))
        assert torch.cuda.current_device() == 0            # the caller's device is left as it was
    finally:
        grp.close()


def test_group_rejects_more_devices_than_present(ops):
    with pytest.raises(ops.LayerOpError):
        ops.HostGroup(torch.cuda.device_count() + 1)
