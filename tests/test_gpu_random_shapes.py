"""Randomised shapes through the launchers (seeded; a few hundred small cases per run): widths that are not vector
multiples, misaligned bases, lane-group / one-CTA / generic kernel selections, partial and gated rotary layouts,
strided rows, every row format of the gather. Each case against the CPU oracle at the usual bar: fp32 1e-5 of the row
maximum (forward_verify's rule, tests/forward_verify.cpp:199-211), bf16 one ulp, integer work bit-exact; plus guard
bands around every output."""
import numpy as np
import pytest
import torch

from util import bf16_ulp_dist, dev, host, max_rel_rows

pytestmark = pytest.mark.gpu
GUARD = 64


def guarded(shape, dtype=torch.float32, fill=-777.0):
    """A CUDA tensor view of `shape` with GUARD elements of `fill` before and after it, and a checker."""
    n = int(np.prod(shape))
    buf = torch.full((n + 2 * GUARD,), fill, device="cuda", dtype=dtype)
    view = buf[GUARD:GUARD + n].view(*shape)

    def intact():
        return bool((buf[:GUARD] == fill).all() and (buf[GUARD + n:] == fill).all())
    return view, intact


def misaligned(a, off):
    """numpy array -> CUDA tensor whose base is `off` elements past a 256-byte boundary."""
    t = torch.zeros(a.size + off + 8, dtype=torch.from_numpy(a).dtype, device="cuda")
    v = t[off:off + a.size].view(*a.shape)
    v.copy_(torch.from_numpy(np.ascontiguousarray(a)))
    return v


def test_add_rmsnorm_random(ops, oracle):
    rng = np.random.default_rng(101)
    widths = [1, 2, 3, 5, 17, 31, 32, 48, 64, 96, 100, 128, 250, 256, 260, 384, 512, 640, 768, 1000, 1024, 1536, 2048, 2560,
              3000, 4096, 5120, 6144, 8192, 8200, 12288]
    for case in range(90):
        n = int(rng.choice(widths))
        T = int(rng.integers(1, 40))
        add, gam, bf16 = rng.random() < 0.5, rng.random() < 0.8, rng.random() < 0.4
        off = int(rng.choice([0, 0, 0, 1, 4]))
        x = rng.standard_normal((T, n)).astype(np.float32) * np.float32(rng.choice([1e-3, 1.0, 30.0]))
        a = rng.standard_normal((T, n)).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32) if gam else None
        if bf16:
            xb, ab = oracle.f32_to_bf16(x).reshape(T, n), oracle.f32_to_bf16(a).reshape(T, n)
            dx = misaligned(xb.view(np.int16), off).view(torch.bfloat16)
            da = misaligned(ab.view(np.int16), off).view(torch.bfloat16) if add else None
            xo, ok1 = guarded((T, n), torch.bfloat16)
            y, ok2 = guarded((T, n), torch.bfloat16)
            ops.gpu_add_rmsnorm(dx, da, xo if add else None, dev(w), y, n, T, 1e-6)
            torch.cuda.synchronize()
            wxo, wy = oracle.add_rmsnorm_bf16(xb, ab if add else None, w, 1e-6)
            assert bf16_ulp_dist(host(y), wy).max() <= 1, (case, n, T, add, gam, off)
            if add:
                assert np.array_equal(host(xo), wxo), (case, n, T)
        else:
            dx, da = misaligned(x, off), misaligned(a, off) if add else None
            xo, ok1 = guarded((T, n))
            y, ok2 = guarded((T, n))
            ops.gpu_add_rmsnorm(dx, da, xo if add else None, dev(w), y, n, T, 1e-6)
            torch.cuda.synchronize()
            wxo, wy = oracle.add_rmsnorm(x, a if add else None, w, 1e-6)
            assert max_rel_rows(host(y), wy) <= 1e-5, (case, n, T, add, gam, off)
            if add:
                assert np.array_equal(host(xo).view(np.uint32), wxo.view(np.uint32)), (case, n, T)
        assert ok1() and ok2(), (case, n, T, add, gam, off)


def test_swiglu_random(ops, oracle):
    rng = np.random.default_rng(102)
    for case in range(60):
        rows, h = int(rng.integers(1, 30)), int(rng.choice([1, 3, 8, 31, 64, 100, 256, 513, 1024, 3072]))
        pad_g, pad_u = int(rng.choice([0, 0, 4, 5, 8])), int(rng.choice([0, 0, 4, 8]))
        bf16 = rng.random() < 0.4
        g = (rng.standard_normal((rows, h + pad_g)) * 3).astype(np.float32)
        u = rng.standard_normal((rows, h + pad_u)).astype(np.float32)
        if bf16:
            gb, ub = oracle.f32_to_bf16(g).reshape(g.shape), oracle.f32_to_bf16(u).reshape(u.shape)
            out, ok = guarded((rows, h), torch.bfloat16)
            ops.gpu_swiglu_rows(dev(gb, torch.bfloat16), dev(ub, torch.bfloat16), out, rows, h, h + pad_g, h + pad_u)
            torch.cuda.synchronize()
            want = oracle.swiglu_bf16(np.ascontiguousarray(gb[:, :h]), np.ascontiguousarray(ub[:, :h])).reshape(rows, h)
            assert bf16_ulp_dist(host(out), want).max() <= 1, (case, rows, h, pad_g, pad_u)
        else:
            out, ok = guarded((rows, h))
            ops.gpu_swiglu_rows(dev(g), dev(u), out, rows, h, h + pad_g, h + pad_u)
            torch.cuda.synchronize()
            want = oracle.swiglu(np.ascontiguousarray(g[:, :h]), np.ascontiguousarray(u[:, :h])).reshape(rows, h)
            assert max_rel_rows(host(out), want) <= 1e-5, (case, rows, h, pad_g, pad_u)
            if pad_g == 0 and pad_u == 0:                       # the flat launcher on the same data: the same bits
                flat, ok3 = guarded((rows * h,))
                ops.gpu_swiglu(dev(g), dev(u), flat, rows * h)
                torch.cuda.synchronize()
                assert torch.equal(flat.view(rows, h), out) and ok3()
        assert ok(), (case, rows, h)


def test_qk_norm_rope_random(ops, oracle):
    rng = np.random.default_rng(103)
    for case in range(70):
        D = int(rng.choice([32, 64, 80, 96, 128, 192, 256, 512]))
        n_rot = int(rng.choice([0, D // 4 // 2 * 2, D // 2, D]))
        rot_pairs = int(rng.choice([0, 0, max(n_rot // 4, 1)])) if n_rot else 0
        n_q, n_kv = int(rng.integers(1, 9)), int(rng.integers(1, 4))
        T = int(rng.choice([1, 2, 3, 4, 5, 7, 16, 33]))
        gated, norm, use_ff, use_pos, bf16 = (rng.random() < p for p in (0.3, 0.85, 0.25, 0.5, 0.4))
        base = float(rng.choice([1e4, 1e6, 1e7]))
        qs = 2 * D if gated else D
        q = rng.standard_normal((T, n_q * qs)).astype(np.float32)
        k = rng.standard_normal((T, n_kv * D)).astype(np.float32)
        qn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32) if rng.random() < 0.8 else None
        kn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32) if rng.random() < 0.8 else None
        ff = (1 + rng.random(max(n_rot // 2, 1))).astype(np.float32) if (use_ff and n_rot) else None
        pos = rng.integers(0, 100000, T).astype(np.int32) if use_pos else None
        pos0 = 0 if use_pos else int(rng.integers(0, 5000))
        tag = (case, D, n_rot, rot_pairs, n_q, n_kv, T, gated, norm, use_ff, use_pos, bf16)
        if bf16:
            qb, kb = oracle.f32_to_bf16(q).reshape(q.shape), oracle.f32_to_bf16(k).reshape(k.shape)
            qo, ok1 = guarded((T, n_q * D), torch.bfloat16)
            ko, ok2 = guarded((T, n_kv * D), torch.bfloat16)
            ops.gpu_qk_norm_rope(dev(qb, torch.bfloat16), dev(kb, torch.bfloat16), dev(qn), dev(kn), qo, ko, n_q, n_kv, D,
                                 n_rot, rot_pairs, dev(pos), pos0, T, base, 1e-6, int(gated), int(norm), dev(ff))
            torch.cuda.synchronize()
            wq, wk = oracle.qk_norm_rope(qb, kb, qn, kn, n_q, n_kv, D, n_rot, rot_pairs, pos, pos0, base, 1e-6,
                                         gated=int(gated), ff=ff, do_norm=int(norm), bf16=True)
            assert bf16_ulp_dist(host(qo), wq).max() <= 1 and bf16_ulp_dist(host(ko), wk).max() <= 1, tag
        else:
            qo, ok1 = guarded((T, n_q * D))
            ko, ok2 = guarded((T, n_kv * D))
            ops.gpu_qk_norm_rope(dev(q), dev(k), dev(qn), dev(kn), qo, ko, n_q, n_kv, D, n_rot, rot_pairs, dev(pos), pos0, T,
                                 base, 1e-6, int(gated), int(norm), dev(ff))
            torch.cuda.synchronize()
            wq, wk = oracle.qk_norm_rope(q, k, qn, kn, n_q, n_kv, D, n_rot, rot_pairs, pos, pos0, base, 1e-6,
                                         gated=int(gated), ff=ff, do_norm=int(norm))
            assert max_rel_rows(host(qo).reshape(-1, D), wq.reshape(-1, D)) <= 1e-5, tag
            assert max_rel_rows(host(ko).reshape(-1, D), wk.reshape(-1, D)) <= 1e-5, tag
        assert ok1() and ok2(), tag


def test_embed_random(ops, oracle):
    from rocm_hip_b200 import synth
    rng = np.random.default_rng(104)
    fmts = [ops.QT_Q8_0, ops.QT_Q4_0, ops.QT_F32, ops.QT_F16, ops.QT_BF16, ops.QT_Q4_1, ops.QT_Q5_0, ops.QT_Q5_1, ops.QT_Q4_K,
            ops.QT_Q5_K, ops.QT_Q6_K]
    for case in range(66):
        qt = fmts[case % len(fmts)]
        blk = ops.QT_BLOCKS[qt][0]
        E = int(rng.choice([256, 512, 768, 1024, 2560, 6400, 7168])) if blk == 256 else int(rng.choice([32, 64, 96, 160, 1024, 5120, 5152, 6400]))
        vocab, T = int(rng.integers(1, 60)), int(rng.integers(1, 70))
        pad = int(rng.choice([0, 0, 2, 6, 16]))
        scale = float(rng.choice([1.0, 1.0, 0.37]))
        table = synth.gguf_table(case, "rnd.%d" % case, qt, vocab, E)
        wide = np.zeros((vocab, table.shape[1] + pad), np.uint8)
        wide[:, :table.shape[1]] = table
        ids = rng.integers(0, vocab, T).astype(np.int32)
        bf16 = rng.random() < 0.5
        out, ok = guarded((T, E), torch.bfloat16 if bf16 else torch.float32)
        flag = ops.gpu_embed_rows(qt, dev(wide), wide.shape[1], vocab, dev(ids), out, E, T, scale)
        torch.cuda.synchronize()
        st, want = oracle.embed_rows(qt, wide, wide.shape[1], vocab, ids, E, scale, bf16=bf16)
        tag = (case, qt, E, vocab, T, pad, scale, bf16)
        assert st == 0 and int(flag.item()) == 2**31 - 1 and ok(), tag
        got = host(out)
        assert np.array_equal(got, want) if bf16 else np.array_equal(got.view(np.uint32), want.view(np.uint32)), tag
