"""gpu_kv_store_f16: K / V rows into the block-major FP16 cache with the reference's row addressing
(src/attention.hip:38-42, src/kv_cache.h:7-14), bit-exact against a numpy statement; and the q/k norm + RoPE -> K row
chain of attn_prep (src/attention.hip:286-299) against the oracle rounded to fp16."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import dev, host

pytestmark = pytest.mark.gpu


def rows_of(pos, kv_stride, kv_shift, kv_bstride):
    pos = np.asarray(pos, dtype=np.int64)
    return (pos >> kv_shift) * kv_bstride + (pos & ((1 << kv_shift) - 1)) * kv_stride


@pytest.mark.parametrize("n_vals,kv_shift,bf16", [(1024, 30, False), (1024, 4, False), (512, 3, True), (200, 2, False),
                                                    (36, 30, True)])
def test_rows_land_where_the_cache_layout_says(ops, oracle, n_vals, kv_shift, bf16):
    T, n_layers = 77, 3
    B = 1 << min(kv_shift, 7)
    kv_stride = n_vals
    kv_bstride = 2 * n_layers * B * n_vals if kv_shift < 30 else 0   # a block holds K and V of every layer
    n_ctx = 256
    size = int(rows_of([n_ctx - 1], kv_stride, kv_shift, kv_bstride)[0]) + n_vals
    src = synth.normal(0, "kv.src", 0, T * n_vals).reshape(T, n_vals) * 4
    want_rows = oracle.f32_to_f16(src)
    d_src = dev(src)
    if bf16:
        b = oracle.f32_to_bf16(src).reshape(T, n_vals)
        want_rows = oracle.f32_to_f16(oracle.bf16_to_f32(b))
        d_src = dev(b, torch.bfloat16)
    for positions, pos0 in ((None, 100), (synth.randint(0, "kv.pos", 0, T, 0, n_ctx).astype(np.int32), 0)):
        if positions is not None:
            positions = np.unique(positions).astype(np.int32)      # distinct rows
        P = positions if positions is not None else np.arange(pos0, pos0 + T)
        n = len(P)
        cache = torch.full((size + 64,), -3.0, device="cuda", dtype=torch.float16)
        ops.gpu_kv_store_f16(d_src, cache, n_vals, dev(positions) if positions is not None else None, pos0, n, kv_stride,
                             kv_shift, kv_bstride)
        torch.cuda.synchronize()
        got = host(cache)
        want = np.full(size + 64, np.float16(-3.0).view(np.uint16), dtype=np.uint16)
        for t, r in enumerate(rows_of(P, kv_stride, kv_shift, kv_bstride)):
            want[r:r + n_vals] = want_rows[t]
        assert np.array_equal(got, want)


def test_attn_prep_chain(ops, oracle):
    """q/k norm + RoPE, then the K row and the V row into the cache, as attn_prep does in one kernel."""
    T, nq, nkv, D, pos0 = 50, 8, 2, 128, 300
    q = synth.normal(0, "ap.q", 0, T * nq * D).reshape(T, nq * D)
    k = synth.normal(0, "ap.k", 0, T * nkv * D).reshape(T, nkv * D)
    v = synth.normal(0, "ap.v", 0, T * nkv * D).reshape(T, nkv * D)
    qn, kn = synth.normal(0, "ap.qn", 0, D, 1.0, 0.1), synth.normal(0, "ap.kn", 0, D, 1.0, 0.1)
    wq, wk = oracle.qk_norm_rope(q, k, qn, kn, nq, nkv, D, D, 0, None, pos0, 1e6, 1e-6)
    dq, dk, dv = dev(q), dev(k), dev(v)
    q_out, k_rot = torch.zeros_like(dq), torch.zeros_like(dk)
    n_ctx, d_kv = 512, nkv * D
    K = torch.zeros(n_ctx * d_kv, device="cuda", dtype=torch.float16)
    V = torch.zeros_like(K)
    ops.gpu_qk_norm_rope(dq, dk, dev(qn), dev(kn), q_out, k_rot, nq, nkv, D, D, 0, None, pos0, T, 1e6, 1e-6)
    ops.gpu_kv_store_f16(k_rot, K, d_kv, None, pos0, T, d_kv, 30, 0)
    ops.gpu_kv_store_f16(dv, V, d_kv, None, pos0, T, d_kv, 30, 0)
    torch.cuda.synchronize()
    assert np.array_equal(host(q_out).view(np.uint32), wq.view(np.uint32))
    assert np.array_equal(host(K).reshape(n_ctx, d_kv)[pos0:pos0 + T], oracle.f32_to_f16(wk).reshape(T, d_kv))
    assert np.array_equal(host(V).reshape(n_ctx, d_kv)[pos0:pos0 + T], oracle.f32_to_f16(v).reshape(T, d_kv))
    assert not host(K).reshape(n_ctx, d_kv)[:pos0].any() and not host(K).reshape(n_ctx, d_kv)[pos0 + T:].any()


def test_argument_errors(ops):
    s = torch.zeros(4, 64, device="cuda")
    c = torch.zeros(4096, device="cuda", dtype=torch.float16)
    for kw in (dict(kv_shift=31), dict(kv_stride=32), dict(T=0), dict(pos0=-1)):
        a = dict(kv_shift=30, kv_stride=64, T=4, pos0=0)
        a.update(kw)
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_kv_store_f16(s, c, 64, None, a["pos0"], a["T"], a["kv_stride"], a["kv_shift"], 0)
        assert e.value.code == 1


def _quant_case(oracle, T, n_vals, bf16):
    src = synth.normal(0, "kvq.src", 0, T * n_vals).reshape(T, n_vals) * 3
    src[1, :32] = 0.0                                   # d == 0: zeros (Q8_0), nibble 8 (Q4_0)
    src[2, 32:64] = np.linspace(-2, 2, 32, dtype=np.float32)   # +- tie of the largest magnitude: the positive one wins
    src[3, 0] = 1e30                                    # one huge value: everything else quantises to the middle
    src[4, 64:96] = -np.abs(src[4, 64:96])              # all negative: d > 0 for Q4_0
    if bf16:
        b = oracle.f32_to_bf16(src).reshape(T, n_vals)
        return oracle.bf16_to_f32(b).reshape(T, n_vals), dev(b, torch.bfloat16)
    return src, dev(src)


@pytest.mark.parametrize("kq", [1, 2])
@pytest.mark.parametrize("n_vals,kv_shift,bf16", [(1024, 30, False), (1024, 4, False), (512, 3, True), (256, 30, True)])
def test_quantised_rows_bit_exact(ops, oracle, kq, n_vals, kv_shift, bf16):
    """Q8_0 / Q4_0 cache rows: values, nibble packing, scales and their place in the row, byte for byte; bytes outside
    the written rows keep their fill."""
    T, n_layers, n_ctx = 61, 2, 256
    B = 1 << min(kv_shift, 7)
    kv_stride = n_vals * (17 if kq == 1 else 9) // 32            # in 2-byte units
    kv_bstride = 2 * n_layers * B * kv_stride if kv_shift < 30 else 0
    size = int(rows_of([n_ctx - 1], kv_stride, kv_shift, kv_bstride)[0]) + kv_stride
    vals, d_src = _quant_case(oracle, T, n_vals, bf16)
    want_q, want_d = oracle.kv_quant_rows(vals, kq)
    vbytes = n_vals if kq == 1 else n_vals // 2
    for positions, pos0 in ((None, 100), (np.unique(synth.randint(0, "kvq.pos", 0, T, 0, n_ctx)).astype(np.int32), 0)):
        P = positions if positions is not None else np.arange(pos0, pos0 + T)
        n = len(P)
        cache = torch.full((size + 64,), 0x5A5A, device="cuda", dtype=torch.int16)
        ops.gpu_kv_store_q(d_src, cache, n_vals, dev(positions) if positions is not None else None, pos0, n, kv_stride,
                           kv_shift, kv_bstride, kq)
        torch.cuda.synchronize()
        got = cache.cpu().numpy().view(np.uint8)
        want = np.full((size + 64) * 2, 0x5A, dtype=np.uint8)
        for t, r in enumerate(rows_of(P, kv_stride, kv_shift, kv_bstride)):
            want[2 * r:2 * r + vbytes] = want_q[t].view(np.uint8)
            want[2 * r + vbytes:2 * r + vbytes + n_vals // 16] = want_d[t].view(np.uint8)
        assert np.array_equal(got, want)


def test_quantised_argument_errors(ops):
    s = torch.zeros(4, 256, device="cuda")
    c = torch.zeros(4096, device="cuda", dtype=torch.int16)
    ok = dict(n_vals=256, kv_stride=136, kq=1)
    for kw in (dict(kq=0), dict(kq=3), dict(n_vals=48), dict(kv_stride=135), dict(kv_stride=72), dict(kq=2, kv_stride=71)):
        a = dict(ok)
        a.update(kw)
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_kv_store_q(s, c, a["n_vals"], None, 0, 4, a["kv_stride"], 30, 0, a["kq"])
        assert e.value.code == 1
    ops.gpu_kv_store_q(s, c, 256, None, 0, 4, 72, 30, 0, 2)     # the Q4_0 row of 256 values is 72 halves
    torch.cuda.synchronize()


@pytest.mark.parametrize("D,N", [(64, 64), (128, 128), (256, 256), (512, 512), (192, 64), (1024, 512), (384, 128)])
def test_hadamard_rotation_is_the_reference_butterfly(ops, oracle, D, N):
    """hadamard_rot (src/attention.hip:251-263): the same butterflies in the same order, so the same bits; its own
    inverse up to rounding; norms preserved; bf16 rows round once."""
    rows = 333
    x = synth.normal(0, "wht.x", 0, rows * D).reshape(rows, D) * 3
    out = torch.empty(rows, D, device="cuda")
    ops.gpu_hadamard_rot(dev(x), out, rows, D, N)
    torch.cuda.synchronize()
    want = oracle.hadamard_rot(x, N)
    assert np.array_equal(host(out).view(np.uint32), want.view(np.uint32))
    back = out.clone()
    ops.gpu_hadamard_rot(back, back, rows, D, N)                       # in place
    torch.cuda.synchronize()
    assert np.abs(host(back) - x).max() <= 2e-5 * np.abs(x).max()
    assert np.allclose(np.linalg.norm(host(out), axis=1), np.linalg.norm(x, axis=1), rtol=1e-5)
    xb = oracle.f32_to_bf16(x).reshape(rows, D)
    ob = torch.empty(rows, D, device="cuda", dtype=torch.bfloat16)
    ops.gpu_hadamard_rot(dev(xb, torch.bfloat16), ob, rows, D, N)
    torch.cuda.synchronize()
    assert np.array_equal(host(ob), oracle.f32_to_bf16(oracle.hadamard_rot(oracle.bf16_to_f32(xb).reshape(rows, D), N)).reshape(rows, D))
    with pytest.raises(ops.LayerOpError):
        ops.gpu_hadamard_rot(dev(x), out, rows, D, 32)


@pytest.mark.parametrize("kq", [1, 2])
@pytest.mark.parametrize("n_vals,rot", [(1024, 128), (1024, 64), (512, 256), (256, 64), (1024, 512), (512, 512)])
def test_rotated_quantised_rows(ops, oracle, kq, n_vals, rot):
    """attn_prep with ATTN_KV_ROT (src/attention.hip:290-295): rotate in blocks, then quantise -- one launch, the bits
    of the rotation followed by the quantiser; and q . k is unchanged when both are rotated."""
    T = 45
    src, d_src = _quant_case(oracle, T, n_vals, False)
    src[3, 0] = 7.0                                                    # (a finite outlier: 1e30 would overflow the sums)
    d_src = dev(src)
    kv_stride = n_vals * (17 if kq == 1 else 9) // 32
    cache = torch.zeros(T * kv_stride, device="cuda", dtype=torch.int16)
    ops.gpu_kv_store_q(d_src, cache, n_vals, None, 0, T, kv_stride, 30, 0, kq, rot_block=rot)
    torch.cuda.synchronize()
    want_q, want_d = oracle.kv_quant_rows(oracle.hadamard_rot(src, rot), kq)
    got = cache.cpu().numpy().view(np.uint8).reshape(T, kv_stride * 2)
    vbytes = n_vals if kq == 1 else n_vals // 2
    assert np.array_equal(got[:, :vbytes], want_q.view(np.uint8).reshape(T, vbytes))
    assert np.array_equal(got[:, vbytes:vbytes + n_vals // 16], want_d.view(np.uint8).reshape(T, n_vals // 16))
    q = synth.normal(0, "wht.q", 0, T * n_vals).reshape(T, n_vals)
    dots = (oracle.hadamard_rot(q, rot).astype(np.float64) * oracle.hadamard_rot(src, rot)).sum(axis=1)
    assert np.allclose(dots, (q.astype(np.float64) * src).sum(axis=1), rtol=1e-4, atol=1e-3)
    with pytest.raises(ops.LayerOpError):
        ops.gpu_kv_store_q(d_src, cache, n_vals, None, 0, T, kv_stride, 30, 0, kq, rot_block=96)


@pytest.mark.parametrize("T,nq,nkv,D,n_rot,kv_shift,bf16,use_pos", [
    (1500, 8, 2, 128, 128, 30, False, False),     # long batch: the trimmed kernel + a tail through the general one
    (1501, 8, 2, 128, 128, 5, True, False),       # bf16, block-major cache, 1 tail token
    (1500, 4, 2, 256, 64, 4, True, True),         # partial rotary, explicit positions
    (37, 8, 4, 128, 128, 3, False, True),         # short batch: the general kernel
    (9, 3, 2, 80, 40, 30, False, False),          # head size without a vector layout: the scalar kernel
    (2000, 16, 8, 64, 64, 30, True, False)])
def test_k_heads_straight_into_the_cache(ops, oracle, T, nq, nkv, D, n_rot, kv_shift, bf16, use_pos):
    """gpu_qk_norm_rope_kv: q as gpu_qk_norm_rope gives it, K rows in the cache exactly as gpu_qk_norm_rope followed by
    gpu_kv_store_f16 leaves them, every other element of the cache untouched."""
    dt = torch.bfloat16 if bf16 else torch.float32
    g = torch.Generator(device="cuda").manual_seed(9)
    q = torch.randn(T, nq * D, device="cuda", generator=g).to(dt)
    k = torch.randn(T, nkv * D, device="cuda", generator=g).to(dt)
    qn, kn = 1 + 0.1 * torch.randn(D, device="cuda", generator=g), 1 + 0.1 * torch.randn(D, device="cuda", generator=g)
    d_kv, layers = nkv * D, 2
    n_ctx = 4096
    B = 1 << min(kv_shift, 12)
    bstride = 2 * layers * B * d_kv if kv_shift < 30 else 0
    size = int(rows_of([n_ctx - 1], d_kv, kv_shift, bstride)[0]) + d_kv
    pos = torch.randperm(n_ctx, device="cuda", generator=g)[:T].to(torch.int32) if use_pos else None
    pos0 = 0 if use_pos else 1000
    fill = torch.full((size,), -3.0, device="cuda", dtype=torch.float16)
    c_sep, c_fused = fill.clone(), fill.clone()
    q1, q2 = torch.empty_like(q), torch.empty_like(q)
    # the two-launch form; for bf16 rows K is taken from the fp32 launcher on the widened inputs, because the fused
    # form rounds K once, to fp16, not to bf16 first
    kf = k.float()
    k1 = torch.empty_like(kf)
    ops.gpu_qk_norm_rope(q, k, qn, kn, q1, torch.empty_like(k), nq, nkv, D, n_rot, 0, pos, pos0, T, 1e6, 1e-6)
    ops.gpu_qk_norm_rope(None, kf, None, kn, None, k1, 0, nkv, D, n_rot, 0, pos, pos0, T, 1e6, 1e-6)
    ops.gpu_kv_store_f16(k1, c_sep, d_kv, pos, pos0, T, d_kv, kv_shift, bstride)
    ops.gpu_qk_norm_rope_kv(q, k, qn, kn, q2, c_fused, d_kv, kv_shift, bstride, nq, nkv, D, n_rot, 0, pos, pos0, T, 1e6, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(q1.view(torch.int16 if bf16 else torch.int32), q2.view(torch.int16 if bf16 else torch.int32))
    if bf16:   # (the bf16 and fp32 kernels sum a head's squares in different orders: 1/rms can differ in its last bit)
        diff = (c_sep.view(torch.int16).int() - c_fused.view(torch.int16).int()).abs()
        assert int(diff.max()) <= 1 and float((diff != 0).float().mean()) < 1e-3
    else:
        assert torch.equal(c_sep.view(torch.int16), c_fused.view(torch.int16))
    touched = int((c_fused != -3.0).sum())
    assert touched >= T * d_kv - 8 and int((c_fused == -3.0).sum()) >= size - T * d_kv     # only the T rows were written
    with pytest.raises(ops.LayerOpError):
        ops.gpu_qk_norm_rope_kv(q, k, qn, kn, q2, c_fused, d_kv - 8, kv_shift, bstride, nq, nkv, D, n_rot, 0, pos, pos0, T, 1e6, 1e-6)
    # the same with the cos / sin read from tables filled once: the same bits in q and in the cache
    ct, st = torch.empty(T, n_rot // 2, device="cuda"), torch.empty(T, n_rot // 2, device="cuda")
    c_tab, q3 = fill.clone(), torch.empty_like(q)
    ops.gpu_rope_table(pos, pos0, T, n_rot, 0, 1e6, ct, st)
    ops.gpu_qk_norm_rope_tab_kv(q, k, qn, kn, q3, c_tab, d_kv, kv_shift, bstride, nq, nkv, D, n_rot, ct, st, pos, pos0, T, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(q3.view(torch.int16 if bf16 else torch.int32), q2.view(torch.int16 if bf16 else torch.int32))
    assert torch.equal(c_tab.view(torch.int16), c_fused.view(torch.int16))


def test_attn_prep_f16_in_one_call(ops, oracle):
    """gpu_attn_prep_f16 against the reference-named attn_prep semantics restated by the oracle: q out, K = fp16 of the
    normed and rotated k, V = fp16 of v, at the rows of the positions (src/attention.hip:266-300)."""
    T, nq, nkv, D, pos0, n_ctx = 130, 8, 2, 128, 40, 512
    q = synth.normal(0, "ap1.q", 0, T * nq * D).reshape(T, nq * D)
    k = synth.normal(0, "ap1.k", 0, T * nkv * D).reshape(T, nkv * D)
    v = synth.normal(0, "ap1.v", 0, T * nkv * D).reshape(T, nkv * D)
    qn, kn = synth.normal(0, "ap1.qn", 0, D, 1.0, 0.1), synth.normal(0, "ap1.kn", 0, D, 1.0, 0.1)
    d_kv = nkv * D
    K = torch.zeros(n_ctx * d_kv, device="cuda", dtype=torch.float16)
    V = torch.zeros_like(K)
    q_out = torch.zeros(T, nq * D, device="cuda")
    ops.gpu_attn_prep_f16(dev(q), dev(k), dev(v), dev(qn), dev(kn), q_out, K, V, d_kv, 30, 0, nq, nkv, D, D, 0, None, pos0, T,
                          1e6, 1e-6)
    torch.cuda.synchronize()
    wq, wk = oracle.qk_norm_rope(q, k, qn, kn, nq, nkv, D, D, 0, None, pos0, 1e6, 1e-6)
    assert np.array_equal(host(q_out).view(np.uint32), wq.view(np.uint32))
    assert np.array_equal(host(K).reshape(n_ctx, d_kv)[pos0:pos0 + T], oracle.f32_to_f16(wk).reshape(T, d_kv))
    assert np.array_equal(host(V).reshape(n_ctx, d_kv)[pos0:pos0 + T], oracle.f32_to_f16(v).reshape(T, d_kv))
    assert not host(K).reshape(n_ctx, d_kv)[:pos0].any() and not host(V).reshape(n_ctx, d_kv)[pos0 + T:].any()
