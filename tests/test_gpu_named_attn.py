"""attn_prep_<D>, the kernels the reference's attention asks its module for by name (src/attention.cpp:55-58), loaded
from rocm_hip_b200/attention.fatbin and launched as src/attention.cpp:150-158 launches them: grid (n_q + n_kv, T),
block D, the 27 arguments of src/attention.hip:970-974. Checked against the CPU oracle (q/k norm + RoPE), a double
precision statement of the flags the oracle does not carry (biases, V norm, interleaved RoPE pairs), and the oracle's
cache-row quantisers and Hadamard rotation."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import dev, host, max_rel_rows

pytestmark = pytest.mark.gpu
FATBIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "rocm_hip_b200", "attention.fatbin")


@pytest.fixture(scope="module")
def prep(ops):
    from cuda.bindings import driver as drv
    torch.zeros(1, device="cuda")
    err, mod = drv.cuModuleLoadData(open(FATBIN, "rb").read())
    assert err == drv.CUresult.CUDA_SUCCESS, err

    def launch(D, T, qfull, k, v, q_norm, k_norm, q_out, K, V, kv_stride, kv_shift, kv_bstride, n_q, n_kv, n_rot, pos0,
               freq_base, eps, gated=0, rot_pairs=None, v_norm=0, qk_norm=1, kv_quant=0, bq=None, bk=None, bv=None,
               rope_norm=0, ff=None):
        err, fn = drv.cuModuleGetFunction(mod, ("attn_prep_%d" % D).encode())
        assert err == drv.CUresult.CUDA_SUCCESS, err
        P = lambda t: C.c_void_p(0 if t is None else t.data_ptr())
        I, F = C.c_int, C.c_float
        args = [P(qfull), P(k), P(v), P(q_norm), P(k_norm), P(q_out), P(K), P(V), I(kv_stride), I(kv_shift),
                C.c_longlong(kv_bstride), I(n_q), I(n_kv), I(n_rot), I(pos0), F(freq_base), F(eps), I(gated),
                I(n_rot // 2 if rot_pairs is None else rot_pairs), I(v_norm), I(qk_norm), I(kv_quant), P(bq), P(bk), P(bv),
                I(rope_norm), P(ff)]
        ptrs = (C.c_void_p * len(args))(*[C.addressof(a) for a in args])
        (err,) = drv.cuLaunchKernel(fn, n_q + n_kv, T, 1, D, 1, 1, 0, torch.cuda.current_stream().cuda_stream,
                                    C.addressof(ptrs), 0)
        assert err == drv.CUresult.CUDA_SUCCESS, err
        torch.cuda.synchronize()

    yield launch
    drv.cuModuleUnload(mod)


def _inputs(T, n_q, n_kv, D, gated):
    qs = 2 * D if gated else D
    q = synth.normal(0, "np.q", 0, T * n_q * qs).reshape(T, n_q * qs)
    k = synth.normal(0, "np.k", 0, T * n_kv * D).reshape(T, n_kv * D)
    v = synth.normal(0, "np.v", 0, T * n_kv * D).reshape(T, n_kv * D)
    qn, kn = synth.normal(0, "np.qn", 0, D, 1.0, 0.1), synth.normal(0, "np.kn", 0, D, 1.0, 0.1)
    return q, k, v, qn, kn


@pytest.mark.parametrize("D,n_q,n_kv,n_rot,rot_pairs,gated,use_ff,kv_shift", [
    (128, 8, 2, 128, None, 0, False, 30), (256, 4, 1, 64, None, 1, False, 4), (64, 6, 2, 64, 20, 0, True, 30),
    (512, 2, 1, 128, None, 0, False, 3), (128, 4, 4, 0, None, 0, False, 30)])
def test_f16_cache(prep, ops, oracle, D, n_q, n_kv, n_rot, rot_pairs, gated, use_ff, kv_shift):
    T, pos0, base, n_ctx = 21, 1000, 1e6, 2048
    q, k, v, qn, kn = _inputs(T, n_q, n_kv, D, gated)
    ff = (1 + np.abs(synth.normal(0, "np.ff", 0, max(n_rot // 2, 1)))).astype(np.float32) if use_ff else None
    d_kv = n_kv * D
    B = 1 << min(kv_shift, 11)
    kv_bstride = 2 * 3 * B * d_kv if kv_shift < 30 else 0
    row = lambda p: (p >> kv_shift) * kv_bstride + (p & ((1 << kv_shift) - 1)) * d_kv
    size = row(n_ctx - 1) + d_kv
    K = torch.full((size,), -3.0, device="cuda", dtype=torch.float16)
    V = torch.full((size,), -3.0, device="cuda", dtype=torch.float16)
    q_out = torch.zeros(T, n_q * D, device="cuda")
    prep(D, T, dev(q), dev(k), dev(v), dev(qn), dev(kn), q_out, K, V, d_kv, kv_shift, kv_bstride, n_q, n_kv, n_rot, pos0,
         base, 1e-6, gated=gated, rot_pairs=rot_pairs, ff=dev(ff))
    wq, wk = oracle.qk_norm_rope(q, k, qn, kn, n_q, n_kv, D, n_rot, 0 if rot_pairs is None else rot_pairs, None, pos0, base,
                                 1e-6, gated=gated, ff=ff)
    assert max_rel_rows(host(q_out).reshape(-1, D), wq.reshape(-1, D)) <= 1e-5
    gK, gV = host(K), host(V)
    wantK, wantV = np.full(size, np.float16(-3.0).view(np.uint16)), np.full(size, np.float16(-3.0).view(np.uint16))
    for t in range(T):
        r = row(pos0 + t)
        wantK[r:r + d_kv] = oracle.f32_to_f16(wk[t])
        wantV[r:r + d_kv] = oracle.f32_to_f16(v[t])
    assert np.array_equal(gV, wantV)
    # K: fp16 of values that agree to 1e-5 -- identical except where a value sits on an fp16 rounding boundary
    assert (gK != wantK).mean() < 1e-3
    assert np.abs(oracle.f16_to_f32(gK).astype(np.float64) - oracle.f16_to_f32(wantK)).max() <= 4e-3


def test_biases_v_norm_and_interleaved_pairs(prep, oracle):
    """bq / bk / bv added first, V normalised without gamma, rope_norm: pairs (2 i, 2 i + 1)
    (src/attention.hip:204-236, 284-292), against the same formulas in double precision."""
    D, n_q, n_kv, T, pos0, base, n_rot = 128, 4, 2, 9, 77, 10000.0, 64
    q, k, v, qn, kn = _inputs(T, n_q, n_kv, D, 0)
    bq, bk, bv = (synth.normal(0, "np.b%d" % i, 0, n * D, 0.0, 0.3) for i, n in enumerate((n_q, n_kv, n_kv)))
    d_kv = n_kv * D
    K = torch.zeros(512 * d_kv, device="cuda", dtype=torch.float16)
    V = torch.zeros_like(K)
    q_out = torch.zeros(T, n_q * D, device="cuda")
    prep(D, T, dev(q), dev(k), dev(v), dev(qn), dev(kn), q_out, K, V, d_kv, 30, 0, n_q, n_kv, n_rot, pos0, base, 1e-6,
         v_norm=1, bq=dev(bq), bk=dev(bk), bv=dev(bv), rope_norm=1)

    def ref(x, b, w, heads, rope=True):
        x = (x + b).astype(np.float64).reshape(T, heads, D)           # fp32 add, then double
        x = x / np.sqrt((x ** 2).mean(axis=2, keepdims=True) + 1e-6)
        if w is not None:
            x = x * w
        if rope:
            i = np.arange(n_rot // 2)
            th = (pos0 + np.arange(T))[:, None, None] * (base ** (-2.0 * i / n_rot))[None, None, :]
            x0, x1 = x[:, :, 0:n_rot:2].copy(), x[:, :, 1:n_rot:2].copy()
            x[:, :, 0:n_rot:2] = x0 * np.cos(th) - x1 * np.sin(th)
            x[:, :, 1:n_rot:2] = x0 * np.sin(th) + x1 * np.cos(th)
        return x.reshape(T, heads * D)

    assert max_rel_rows(host(q_out).reshape(-1, D), ref(q, bq, qn, n_q).reshape(-1, D)) <= 1e-5
    gK = oracle.f16_to_f32(host(K)).reshape(512, d_kv)[pos0:pos0 + T]
    gV = oracle.f16_to_f32(host(V)).reshape(512, d_kv)[pos0:pos0 + T]
    assert np.abs(gK - ref(k, bk, kn, n_kv)).max() <= 4e-3 and np.abs(gV - ref(v, bv, None, n_kv, rope=False)).max() <= 4e-3


@pytest.mark.parametrize("kq", [1, 2])
@pytest.mark.parametrize("rot", [0, 4])
@pytest.mark.parametrize("D,n_kv", [(128, 2), (256, 1), (512, 1), (64, 4)])
def test_quantised_cache_rows(prep, oracle, kq, rot, D, n_kv):
    """Q8_0 / Q4_0 rows with and without ATTN_KV_ROT (src/attention.hip:290-296). Without RoPE the K values are the
    oracle's to the bit, so the rows are compared byte for byte: quantiser(rotation(norm(k))), and q_out rotated."""
    n_q, T, pos0 = 2 * n_kv, 11, 5
    q, k, v, qn, kn = _inputs(T, n_q, n_kv, D, 0)
    d_kv = n_kv * D
    kv_stride = d_kv * (17 if kq == 1 else 9) // 32
    K = torch.zeros(64 * kv_stride, device="cuda", dtype=torch.int16)
    V = torch.zeros_like(K)
    q_out = torch.zeros(T, n_q * D, device="cuda")
    prep(D, T, dev(q), dev(k), dev(v), dev(qn), dev(kn), q_out, K, V, kv_stride, 30, 0, n_q, n_kv, 0, pos0, 1e6, 1e-6,
         kv_quant=kq | rot)
    wq, wk = oracle.qk_norm_rope(q, k, qn, kn, n_q, n_kv, D, 0, 0, None, pos0, 1e6, 1e-6)
    wv = v
    if rot:
        N = oracle.hadamard_k(D)
        wq = oracle.hadamard_rot(wq.reshape(-1, D), N).reshape(wq.shape)
        wk = oracle.hadamard_rot(wk.reshape(-1, D), N).reshape(wk.shape)
        wv = oracle.hadamard_rot(v.reshape(-1, D), 64).reshape(v.shape)
    assert np.array_equal(host(q_out).view(np.uint32), wq.view(np.uint32))
    vbytes = d_kv if kq == 1 else d_kv // 2
    for cache, vals in ((K, wk), (V, wv)):
        want_q, want_d = oracle.kv_quant_rows(vals, kq)
        got = cache.cpu().numpy().view(np.uint8).reshape(64, kv_stride * 2)[pos0:pos0 + T]
        assert np.array_equal(got[:, :vbytes], want_q.view(np.uint8).reshape(T, vbytes))
        assert np.array_equal(got[:, vbytes:vbytes + d_kv // 16], want_d.view(np.uint8).reshape(T, d_kv // 16))
