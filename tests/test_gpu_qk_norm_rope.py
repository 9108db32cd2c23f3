"""CUDA per-head q/k RMSNorm + NeoX RoPE against the CPU oracle through the C ABI. fp32: worst head row of
max|d|/max|ref| <= 1e-5 (a per-element relative error is meaningless for rotated values that cancel to ~0).
bf16: within 1 bf16 ulp."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import bf16_ulp_dist, dev, host, max_rel_rows

pytestmark = pytest.mark.gpu


def run(ops, oracle, T, nq, nkv, D, n_rot, base, positions=None, pos0=0, gated=0, rot_pairs=0, ff=None, qk_norm=1,
        bf16=False, seed=0, gamma=True, inplace=False):
    qs = 2 * D if gated else D
    q = synth.normal(seed, "qk.q", 0, T * nq * qs).reshape(T, nq * qs)
    k = synth.normal(seed, "qk.k", 0, T * nkv * D).reshape(T, nkv * D)
    qn = synth.normal(seed, "qk.qn", 0, D, 1.0, 0.1) if gamma else None
    kn = synth.normal(seed, "qk.kn", 0, D, 1.0, 0.1) if gamma else None
    dt = None
    if bf16:
        q, k, dt = oracle.f32_to_bf16(q).reshape(q.shape), oracle.f32_to_bf16(k).reshape(k.shape), torch.bfloat16
    wq, wk = oracle.qk_norm_rope(q, k, qn, kn, nq, nkv, D, n_rot, rot_pairs, positions, pos0, base, 1e-6, gated=gated,
                                 ff=ff, do_norm=qk_norm, bf16=bf16)
    dq, dk = dev(q, dt), dev(k, dt)
    if inplace:
        qo, ko = dq, dk
    else:
        qo = torch.zeros(T, nq * D, device="cuda", dtype=dq.dtype)
        ko = torch.zeros(T, nkv * D, device="cuda", dtype=dq.dtype)
    ops.gpu_qk_norm_rope(dq, dk, dev(qn), dev(kn), qo, ko, nq, nkv, D, n_rot, rot_pairs,
                         dev(positions) if positions is not None else None, pos0, T, base, 1e-6, gated, qk_norm, dev(ff))
    torch.cuda.synchronize()
    gq, gk = host(qo), host(ko)
    if bf16:
        return max(bf16_ulp_dist(gq, wq).max(initial=0), bf16_ulp_dist(gk, wk).max(initial=0))
    return max(max_rel_rows(gq.reshape(-1, D), wq.reshape(-1, D)), max_rel_rows(gk.reshape(-1, D), wk.reshape(-1, D)))


def test_c1_fp32(ops, oracle):
    """Qwen3-0.6B: 2,427 tokens, 16 Q + 8 KV heads of 128, theta 1e6, positions 0..2426."""
    assert run(ops, oracle, 2427, 16, 8, 128, 128, 1e6) <= 1e-5


def test_c2_decode_bf16(ops, oracle):
    """64 sequences x 1 token, positions uniform in [0, 32768)."""
    pos = synth.randint(0, "c2.pos", 0, 64, 0, 32768).astype(np.int32)
    assert run(ops, oracle, 64, 16, 8, 128, 128, 1e6, positions=pos, bf16=True) <= 1
    assert run(ops, oracle, 64, 16, 8, 128, 128, 1e6, positions=pos) <= 1e-5


def test_c3_partial_rotary_gated_bf16(ops, oracle):
    """Qwen3.5-4B-like: head_dim 256, rotary over the first 64 dims, theta 1e7, 16 Q (gated stride) + 4 KV heads."""
    assert run(ops, oracle, 1024, 16, 4, 256, 64, 1e7, gated=1, bf16=True) <= 1
    assert run(ops, oracle, 512, 16, 4, 256, 64, 1e7, gated=1) <= 1e-5


def test_c5_heads_and_far_positions(ops, oracle):
    """27B shape (40 Q + 8 KV heads of 128) at the last positions of a 262,144-token prefill: the angle is formed
    in double precision, so 1e-5 holds where an fp32 angle is off by ~0.03 rad."""
    assert run(ops, oracle, 96, 40, 8, 128, 128, 1e6, pos0=262144 - 96) <= 1e-5
    assert run(ops, oracle, 96, 40, 8, 128, 128, 1e6, pos0=262144 - 96, bf16=True) <= 1
    pos = np.array([0, 1, 2499, 131072, 262143, 1 << 24, (1 << 30) + 12345], dtype=np.int32)
    assert run(ops, oracle, pos.size, 4, 2, 128, 128, 1e6, positions=pos) <= 1e-5


@pytest.mark.parametrize("pos0", [0, 123456789, 2**30, 2**31 - 1501])
def test_tile_kernel_trig_over_the_whole_position_range(ops, oracle, pos0):
    """Long batches take the tile kernel, which evaluates sin / cos itself (Cody-Waite reduction with exact products
    for every int32 position): 1e-5 must hold from position 0 to the last int32 position, fp32 and bf16, and the
    results are in fact the CPU reference's bits (a handful of last-bit differences would still be legitimate)."""
    T, nq, nkv, D = 1500, 4, 2, 128
    q = synth.normal(9, "far.q", 0, T * nq * D).reshape(T, nq * D)
    k = synth.normal(9, "far.k", 0, T * nkv * D).reshape(T, nkv * D)
    qn, kn = synth.normal(9, "far.qn", 0, D, 1.0, 0.1), synth.normal(9, "far.kn", 0, D, 1.0, 0.1)
    wq, wk = oracle.qk_norm_rope(q, k, qn, kn, nq, nkv, D, D, 0, None, pos0, 1e6, 1e-6)
    qo, ko = torch.zeros(T, nq * D, device="cuda"), torch.zeros(T, nkv * D, device="cuda")
    ops.gpu_qk_norm_rope(dev(q), dev(k), dev(qn), dev(kn), qo, ko, nq, nkv, D, D, 0, None, pos0, T, 1e6, 1e-6)
    torch.cuda.synchronize()
    assert max_rel_rows(host(qo).reshape(-1, D), wq.reshape(-1, D)) <= 1e-5
    assert max_rel_rows(host(ko).reshape(-1, D), wk.reshape(-1, D)) <= 1e-5
    differing = int((host(qo).view(np.uint32) != wq.view(np.uint32)).sum())
    assert differing <= 8, differing
    assert run(ops, oracle, T, nq, nkv, D, D, 1e6, pos0=pos0, bf16=True, seed=9) <= 1


@pytest.mark.parametrize("D,n_rot", [(64, 64), (128, 64), (128, 128), (256, 256), (512, 512), (512, 128), (96, 32),
                                     (80, 80), (128, 20), (256, 0)])
def test_head_shapes(ops, oracle, D, n_rot):
    """Vector paths (power-of-two heads), the two-pairs-per-thread path (512), and the generic path (96, 80, a rotary
    width that is not whole vectors, no rotation at all)."""
    for bf16 in (False, True):
        r = run(ops, oracle, 33, 5, 3, D, n_rot, 1e4, pos0=1000, bf16=bf16, seed=D + n_rot)
        assert r <= (1 if bf16 else 1e-5)


def test_options(ops, oracle):
    """rot_pairs < n_rot/2, frequency factors, no gamma, no norm (RoPE only), Q only / K only, in place."""
    ff = (1.0 + synth.uniform(0, "ff", 0, 64) * 7).astype(np.float32)
    assert run(ops, oracle, 50, 8, 2, 128, 128, 1e6, rot_pairs=24, pos0=77) <= 1e-5
    assert run(ops, oracle, 50, 8, 2, 128, 128, 5e5, ff=ff, pos0=4000) <= 1e-5
    assert run(ops, oracle, 50, 8, 2, 128, 128, 1e6, gamma=False, pos0=9) <= 1e-5
    assert run(ops, oracle, 50, 8, 2, 128, 128, 1e6, qk_norm=0, pos0=9) <= 1e-5
    assert run(ops, oracle, 50, 8, 0, 128, 128, 1e6, pos0=9) <= 1e-5
    assert run(ops, oracle, 50, 0, 2, 128, 128, 1e6, pos0=9, bf16=True) <= 1
    assert run(ops, oracle, 50, 8, 2, 128, 128, 1e6, pos0=9, inplace=True) <= 1e-5
    assert run(ops, oracle, 50, 8, 2, 96, 96, 1e6, pos0=9, inplace=True) <= 1e-5
    assert run(ops, oracle, 2000, 40, 8, 128, 128, 1e6, pos0=9, inplace=True, bf16=True) <= 1


def run_tab(ops, oracle, T, nq, nkv, D, n_rot, base, positions=None, pos0=0, gated=0, rot_pairs=0, ff=None, qk_norm=1,
            bf16=False, seed=0):
    """The table route: gpu_rope_table once, then gpu_qk_norm_rope_tab; checked like run()."""
    qs = 2 * D if gated else D
    q = synth.normal(seed, "qk.q", 0, T * nq * qs).reshape(T, nq * qs)
    k = synth.normal(seed, "qk.k", 0, T * nkv * D).reshape(T, nkv * D)
    qn, kn = synth.normal(seed, "qk.qn", 0, D, 1.0, 0.1), synth.normal(seed, "qk.kn", 0, D, 1.0, 0.1)
    dt = None
    if bf16:
        q, k, dt = oracle.f32_to_bf16(q).reshape(q.shape), oracle.f32_to_bf16(k).reshape(k.shape), torch.bfloat16
    wq, wk = oracle.qk_norm_rope(q, k, qn, kn, nq, nkv, D, n_rot, rot_pairs, positions, pos0, base, 1e-6, gated=gated,
                                 ff=ff, do_norm=qk_norm, bf16=bf16)
    dq, dk = dev(q, dt), dev(k, dt)
    qo = torch.zeros(T, nq * D, device="cuda", dtype=dq.dtype)
    ko = torch.zeros(T, nkv * D, device="cuda", dtype=dq.dtype)
    ct = torch.full((T, max(n_rot // 2, 1)), 7.0, device="cuda")
    st = torch.full((T, max(n_rot // 2, 1)), 7.0, device="cuda")
    ops.gpu_rope_table(dev(positions) if positions is not None else None, pos0, T, n_rot, rot_pairs, base, ct, st, dev(ff))
    ops.gpu_qk_norm_rope_tab(dq, dk, dev(qn), dev(kn), qo, ko, nq, nkv, D, n_rot, ct, st, T, 1e-6, gated, qk_norm)
    torch.cuda.synchronize()
    gq, gk = host(qo), host(ko)
    if bf16:
        return max(bf16_ulp_dist(gq, wq).max(initial=0), bf16_ulp_dist(gk, wk).max(initial=0))
    return max(max_rel_rows(gq.reshape(-1, D), wq.reshape(-1, D)), max_rel_rows(gk.reshape(-1, D), wk.reshape(-1, D)))


def test_table_route_on_the_config_shapes(ops, oracle):
    """cos / sin from gpu_rope_table + gpu_qk_norm_rope_tab against the CPU oracle: c1 (fp32), c2 (per-row
    positions), c3 (gated q, partial rotary, theta 1e7), c5 heads at the far end of a 262,144-token prefill; short
    batches (general kernel) and long ones (tile kernel with asynchronous table copies, plus its tail tokens)."""
    assert run_tab(ops, oracle, 2427, 16, 8, 128, 128, 1e6) <= 1e-5
    pos = synth.randint(0, "c2.pos", 0, 64, 0, 32768).astype(np.int32)
    assert run_tab(ops, oracle, 64, 16, 8, 128, 128, 1e6, positions=pos, bf16=True) <= 1
    assert run_tab(ops, oracle, 1500, 16, 4, 256, 64, 1e7, gated=1, bf16=True) <= 1
    assert run_tab(ops, oracle, 1499, 16, 4, 256, 64, 1e7, gated=1) <= 1e-5
    assert run_tab(ops, oracle, 1501, 40, 8, 128, 128, 1e6, pos0=262144 - 1501) <= 1e-5
    assert run_tab(ops, oracle, 1501, 40, 8, 128, 128, 1e6, pos0=262144 - 1501, bf16=True) <= 1


def test_table_route_options_and_head_shapes(ops, oracle):
    """rot_pairs < n_rot / 2, frequency factors, RoPE only, the generic path (96), no rotation at all."""
    ff = (1.0 + synth.uniform(0, "ff", 0, 64) * 7).astype(np.float32)
    assert run_tab(ops, oracle, 50, 8, 2, 128, 128, 1e6, rot_pairs=24, pos0=77) <= 1e-5
    assert run_tab(ops, oracle, 1300, 8, 2, 128, 128, 1e6, rot_pairs=24, pos0=77) <= 1e-5
    assert run_tab(ops, oracle, 50, 8, 2, 128, 128, 5e5, ff=ff, pos0=4000) <= 1e-5
    assert run_tab(ops, oracle, 50, 8, 2, 128, 128, 1e6, qk_norm=0, pos0=9) <= 1e-5
    for D, n_rot in ((64, 64), (512, 512), (512, 128), (96, 32), (128, 20), (256, 0)):
        for bf16 in (False, True):
            r = run_tab(ops, oracle, 33, 5, 3, D, n_rot, 1e4, pos0=1000, bf16=bf16, seed=D + n_rot)
            assert r <= (1 if bf16 else 1e-5), (D, n_rot, bf16, r)


def test_table_route_gives_the_bits_of_the_direct_route(ops):
    """On a long batch both routes evaluate sin / cos with the same routine, so the outputs are identical; the table
    itself holds (1, 0) beyond rot_pairs."""
    T, nq, nkv, D = 1400, 8, 2, 128
    q, k = torch.randn(T, nq * D, device="cuda"), torch.randn(T, nkv * D, device="cuda")
    w = 1 + 0.1 * torch.randn(D, device="cuda")
    for dt in (torch.float32, torch.bfloat16):
        qq, kk = q.to(dt), k.to(dt)
        a = [torch.empty_like(qq), torch.empty_like(kk)]
        b = [torch.empty_like(qq), torch.empty_like(kk)]
        ops.gpu_qk_norm_rope(qq, kk, w, w, a[0], a[1], nq, nkv, D, D, 40, None, 1000, T, 1e6, 1e-6)
        ct, st = torch.empty(T, D // 2, device="cuda"), torch.empty(T, D // 2, device="cuda")
        ops.gpu_rope_table(None, 1000, T, D, 40, 1e6, ct, st)
        ops.gpu_qk_norm_rope_tab(qq, kk, w, w, b[0], b[1], nq, nkv, D, D, ct, st, T, 1e-6)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
        assert bool((ct[:, 40:] == 1).all()) and bool((st[:, 40:] == 0).all())
    with pytest.raises(ops.LayerOpError):
        ops.gpu_qk_norm_rope_tab(q, k, w, w, a[0], a[1], nq, nkv, D, D, None, None, T, 1e-6)


def test_rope_alone_matches_golden(ops):
    """qk_norm 0 on the reference's own outputs (tests/golden/rope_neox.npz, made by qwen_rope_neox)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rope_neox.npz"))
    pos = g["positions"]
    for name, D, n_rot, base in (("d128_full_1e6", 128, 128, 1e6), ("d256_rot64_1e7", 256, 64, 1e7),
                                  ("d64_full_1e4", 64, 64, 1e4)):
        x, want = g[name + "_x"], g[name + "_y"]
        dq = dev(x)
        out = torch.zeros_like(dq)
        ops.gpu_qk_norm_rope(dq, None, None, None, out, None, 1, 0, D, n_rot, 0, dev(pos), 0, pos.size, base, 1e-6, 0, 0)
        torch.cuda.synchronize()
        assert max_rel_rows(host(out), want) <= 1e-6


def test_positions_give_same_bits_as_pos0(ops):
    T = 300
    q = torch.randn(T, 8 * 128, device="cuda")
    k = torch.randn(T, 2 * 128, device="cuda")
    w = torch.ones(128, device="cuda")
    a = [torch.empty_like(q), torch.empty_like(k)]
    b = [torch.empty_like(q), torch.empty_like(k)]
    ops.gpu_qk_norm_rope(q, k, w, w, a[0], a[1], 8, 2, 128, 128, 0, None, 40, T, 1e6, 1e-6)
    pos = torch.arange(40, 40 + T, dtype=torch.int32, device="cuda")
    ops.gpu_qk_norm_rope(q, k, w, w, b[0], b[1], 8, 2, 128, 128, 0, pos, 0, T, 1e6, 1e-6)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    # a shard of the rows gives the rows' bits
    c = [torch.empty(100, 8 * 128, device="cuda"), torch.empty(100, 2 * 128, device="cuda")]
    ops.gpu_qk_norm_rope(q[200:], k[200:], w, w, c[0], c[1], 8, 2, 128, 128, 0, pos[200:], 0, 100, 1e6, 1e-6)
    assert torch.equal(c[0], a[0][200:]) and torch.equal(c[1], a[1][200:])


def test_argument_errors(ops):
    q = torch.randn(4, 2 * 128, device="cuda")
    for kwargs in (dict(n_rot=130), dict(n_rot=127), dict(rot_pairs=65), dict(T=0), dict(pos0=-1), dict(D=2048)):
        args = dict(n_rot=128, rot_pairs=0, T=4, pos0=0, D=128)
        args.update(kwargs)
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_qk_norm_rope(q, None, None, None, q, None, 2, 0, args["D"], args["n_rot"], args["rot_pairs"], None,
                                 args["pos0"], args["T"], 1e6, 1e-6)
        assert e.value.code == 1


def test_fp16_rope_component_sweep(ops, oracle):
    """The reference's rope_verify sweep (tests/rope_verify.cpp:69-93,152-164) through gpu_rope_rotate_half_f16:
    identical tables, identical algebra, so the result is the restated CPU loop's to the bit; in place too."""
    state, positions = 99, []
    for _ in range(64):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        positions.append(1 + (state >> 8) % 4096)
    positions = np.array(positions, dtype=np.int32)
    for rows, dim in ((16, 16), (5, 32), (64, 128), (7, 6)):
        rng = oracle.Lcg(13)
        x = oracle.f32_to_f16(np.array([rng.rnd(-3.0, 3.0) for _ in range(rows * dim)], dtype=np.float32)).reshape(rows, dim)
        c, s = oracle.rope_tables(positions[:rows], dim, 10000.0)
        want = oracle.rope_rotate_half_f16(x, c, s)
        dx = dev(x, torch.float16)
        dy = torch.zeros_like(dx)
        ops.gpu_rope_rotate_half_f16(dx, dev(c), dev(s), dy, rows, dim // 2)
        ops.gpu_rope_rotate_half_f16(dx, dev(c), dev(s), dx, rows, dim // 2)
        torch.cuda.synchronize()
        assert np.array_equal(host(dy), want) and np.array_equal(host(dx), want)
