"""The sibling chains of the reference's Gemma-4 layers behind their reference-named launchers (src/gpu_ops.h:48-68):
gpu_add_normed, gpu_gemma_attn_post, gpu_geglu, gpu_softcap against the oracle's statement of the kernels'
arithmetic (src/gpu_ops.hip:521-606, 659-677), and the chains against the separate kernels they fuse."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import dev, host, max_rel_rows

pytestmark = pytest.mark.gpu

WIDTHS = [256, 768, 1024, 2816, 3840, 4096]      # n % 256 == 0, both vector-per-thread plans


@pytest.mark.parametrize("n", WIDTHS)
def test_add_normed(ops, oracle, n):
    T = 37
    base = synth.normal(1, "an.b", 0, T * n).reshape(T, n)
    a = synth.normal(1, "an.a", 0, T * n).reshape(T, n) * 3
    w = synth.normal(1, "an.w", 0, n, 1.0, 0.1)
    db, da, dw = dev(base), dev(a), dev(w)
    for scale in (None, 0.625, 1.7):
        out = torch.empty_like(db)
        ds = None if scale is None else torch.tensor([scale], device="cuda", dtype=torch.float32)
        ops.gpu_add_normed(db, da, dw, ds, out, n, T, 1e-6)
        torch.cuda.synchronize()
        want = oracle.add_normed(base, a, w, scale, 1e-6)
        assert np.array_equal(host(out).view(np.uint32), want.view(np.uint32))
    # out may be base; and the chain is the norm kernel followed by an fp32 add
    y = torch.empty_like(db)
    ops.gpu_add_rmsnorm(da, None, da, dw, y, n, T, 1e-6)
    inplace = db.clone()
    ops.gpu_add_normed(inplace, da, dw, None, inplace, n, T, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(inplace, db + y)


@pytest.mark.parametrize("n", WIDTHS)
@pytest.mark.parametrize("router", [False, True])
def test_gemma_attn_post(ops, oracle, n, router):
    T = 29
    x = synth.normal(2, "ap.x", 0, T * n).reshape(T, n)
    a = synth.normal(2, "ap.a", 0, T * n).reshape(T, n) * 2
    w_a, w1, w2 = (synth.normal(2, "ap.w%d" % i, 0, n, 1.0, 0.1) for i in range(3))
    dx, da = dev(x), dev(a)
    x_out, y1, y2 = torch.empty_like(dx), torch.empty_like(dx), torch.full_like(dx, -7.0)
    q8 = ops.Q8Buffers(T * n, "cuda", xh="bf16")
    ops.gpu_gemma_attn_post(dx, da, dev(w_a), x_out, dev(w1), y1, dev(w2) if router else None, y2 if router else None,
                            n, T, 1e-6, q8=q8)
    torch.cuda.synchronize()
    wx, wy1, wy2 = oracle.gemma_attn_post(x, a, w_a, w1, w2 if router else None, 1e-6)
    assert np.array_equal(host(x_out).view(np.uint32), wx.view(np.uint32))
    assert np.array_equal(host(y1).view(np.uint32), wy1.view(np.uint32))
    if router:
        assert np.array_equal(host(y2).view(np.uint32), wy2.view(np.uint32))
    else:
        assert (host(y2) == -7.0).all()
    want = oracle.quantize_q8(host(y1), xh="bf16")          # the side outputs of y1 (src/gpu_ops.hip:603)
    for k in ("q0", "d0", "s0", "qK", "dK", "bsK"):
        assert np.array_equal(host(getattr(q8, k)).view(want[k].dtype), want[k]), k
    assert np.array_equal(host(q8.xh).view(np.uint16), want["xh"])
    # the same bits as the separate kernels: add_normed, then the plain norm (src/gpu_ops.hip:552-554)
    sx, sy = torch.empty_like(dx), torch.empty_like(dx)
    ops.gpu_add_normed(dx, da, dev(w_a), None, sx, n, T, 1e-6)
    ops.gpu_add_rmsnorm(sx, None, sx, dev(w1), sy, n, T, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(sx, x_out) and max_rel_rows(host(sy), host(y1)) <= 1e-6


@pytest.mark.parametrize("rows,h,gs,us,fused", [(33, 704, 704, 704, False), (50, 512, 1024, 1024, True),
                                                (7, 100, 100, 100, False), (5, 37, 80, 80, True)])
def test_geglu(ops, oracle, rows, h, gs, us, fused):
    if fused:                                    # the experts' rows [gate h | up h ...], up = gate + h
        buf = synth.normal(3, "gg.b", 0, rows * gs).reshape(rows, gs) * 2
        d = dev(buf)
        gate, up, dg, du = buf[:, :h], buf[:, h:2 * h], d, d[:, h:]
    else:
        gate = synth.normal(3, "gg.g", 0, rows * h).reshape(rows, h) * 2
        up = synth.normal(3, "gg.u", 0, rows * h).reshape(rows, h)
        dg, du = dev(gate), dev(up)
    out = torch.empty(rows, h, device="cuda")
    ops.gpu_geglu(dg, du, out, rows, h, gs, us)
    torch.cuda.synchronize()
    want = oracle.geglu(gate, up)
    assert max_rel_rows(host(out), want) <= 1e-5
    assert np.abs(host(out) - want).max() <= 1e-6 * max(1.0, np.abs(want).max())


def test_geglu_side_outputs_and_errors(ops, oracle):
    rows, h = 8, 256
    g, u = synth.normal(3, "gq.g", 0, rows * h), synth.normal(3, "gq.u", 0, rows * h)
    q8 = ops.Q8Buffers(rows * h, "cuda", xh="f16")
    out = torch.empty(rows * h, device="cuda")
    ops.gpu_geglu(dev(g), dev(u), out, rows, h, h, h, q8=q8)
    torch.cuda.synchronize()
    want = oracle.quantize_q8(host(out), xh="f16")
    for k in ("q0", "d0", "s0", "qK", "dK", "bsK"):
        assert np.array_equal(host(getattr(q8, k)).view(want[k].dtype), want[k]), k
    assert np.array_equal(host(q8.xh).view(np.uint16), want["xh"])
    for kw in (dict(rows=0), dict(h=0), dict(gs=h - 1), dict(us=h - 1)):
        a = dict(rows=rows, h=h, gs=h, us=h)
        a.update(kw)
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_geglu(dev(g), dev(u), out, a["rows"], a["h"], a["gs"], a["us"])
        assert e.value.code == 1
    with pytest.raises(ops.LayerOpError):
        ops.gpu_geglu(dev(g), dev(u), out, rows - 1, h - 1, h, h, q8=q8)        # n % 32 != 0 with q8


@pytest.mark.parametrize("n", [1, 7, 4096, 262144 + 3])
def test_softcap(ops, oracle, n):
    x = synth.normal(4, "sc.x", 0, n) * 40
    for cap in (30.0, 50.0):
        d = dev(x)
        ops.gpu_softcap(d, n, cap)
        torch.cuda.synchronize()
        want = oracle.softcap(x, cap)
        assert np.abs(host(d) - want).max() <= 4e-6 * cap and np.abs(host(d)).max() <= cap
    with pytest.raises(ops.LayerOpError):
        ops.gpu_softcap(dev(x), n, 0.0)
    with pytest.raises(ops.LayerOpError):
        ops.gpu_softcap(dev(x), 0, 30.0)


def test_chain_argument_errors(ops):
    """src/gpu_ops.cpp:189,198: T <= 0, n % 256 != 0, n > 4096, a == out; x_out == x or a."""
    t = lambda n, T=4: torch.zeros(T, n, device="cuda")
    w = torch.ones(8192, device="cuda")
    for n, T in ((255, 4), (4352, 4), (512, 0)):
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_add_normed(t(n), t(n), w, None, t(n), n, T, 1e-6)
        assert e.value.code == 1
    a = t(512)
    with pytest.raises(ops.LayerOpError):
        ops.gpu_add_normed(t(512), a, w, None, a, 512, 4, 1e-6)
    x = t(512)
    for xo in (x, a):
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_gemma_attn_post(x, a, w, xo, w, t(512), None, None, 512, 4, 1e-6)
        assert e.value.code == 1
    small = ops.Q8Buffers(256, "cuda")
    with pytest.raises(ops.LayerOpError):
        ops.gpu_gemma_attn_post(x, a, w, t(512), w, t(512), None, None, 512, 4, 1e-6, q8=small)


def _moe_case(T, n_used, n, n_expert, seed):
    down = synth.normal(seed, "mc.d", 0, T * n_used * n).reshape(T, n_used, n)
    wts = np.abs(synth.normal(seed, "mc.w", 0, T * n_used)).reshape(T, n_used).astype(np.float32)
    wts /= wts.sum(axis=1, keepdims=True)
    ids = synth.randint(seed, "mc.i", 0, T * n_used, 0, n_expert).astype(np.int32).reshape(T, n_used)
    es = synth.normal(seed, "mc.e", 0, n_expert, 1.0, 0.2)
    return down, wts.astype(np.float32), ids, es


@pytest.mark.parametrize("T,n_used,n", [(19, 8, 2048), (7, 10, 1000), (5, 3, 37), (3, 1, 256), (4, 17, 512)])
def test_moe_combine(ops, oracle, T, n_used, n):
    """Every variant of src/gpu_ops.hip:245-264 bit for bit: weighted, per-expert scales, gated / ungated shared
    expert, weight 1."""
    down, wts, ids, es = _moe_case(T, n_used, n, 64, 5)
    shared = synth.normal(5, "mc.s", 0, T * n).reshape(T, n)
    sg = synth.normal(5, "mc.g", 0, T, 0.5, 0.1)
    dd, dw, di, de, dsh, dsg = dev(down), dev(wts), dev(ids), dev(es), dev(shared), dev(sg)
    cases = [dict(wts=wts), dict(wts=wts, shared=shared, sg=sg), dict(wts=wts, shared=shared),
             dict(wts=wts, ids=ids, exp_scale=es), dict(wts=wts, ids=ids, exp_scale=es, shared=shared, sg=sg),
             dict(wts=None), dict(wts=None, shared=shared, sg=sg)]
    for kw in cases:
        out = torch.full((T, n), -1.0, device="cuda")
        ops.gpu_moe_combine(dd, dw if kw.get("wts") is not None else None, dsh if "shared" in kw else None,
                            dsg if "sg" in kw else None, out, n_used, n, T, di if "ids" in kw else None,
                            de if "exp_scale" in kw else None)
        torch.cuda.synchronize()
        want = oracle.moe_combine(down, kw.get("wts"), kw.get("shared"), kw.get("sg"), kw.get("ids"), kw.get("exp_scale"))
        assert np.array_equal(host(out).view(np.uint32), want.view(np.uint32)), sorted(kw)
    with pytest.raises(ops.LayerOpError) as e:      # exp_scale without ids (src/gpu_ops.cpp:108)
        ops.gpu_moe_combine(dd, dw, None, None, torch.empty(T, n, device="cuda"), n_used, n, T, None, de)
    assert e.value.code == 1


@pytest.mark.parametrize("n", [256, 1536, 2816, 4096])
@pytest.mark.parametrize("scaled", [False, True])
def test_gemma_ffn_post(ops, oracle, n, scaled):
    T, n_used = 23, 8
    down, wts, ids, es = _moe_case(T, n_used, n, 128, 6)
    x = synth.normal(6, "fp.x", 0, T * n).reshape(T, n)
    mlp = synth.normal(6, "fp.m", 0, T * n).reshape(T, n) * 2
    w1, w2, w_post, w_next = (synth.normal(6, "fp.w%d" % i, 0, n, 1.0, 0.1) for i in range(4))
    scale = 0.8125 if scaled else None
    ds = torch.tensor([scale], device="cuda") if scaled else None
    x_out, y = torch.empty(T, n, device="cuda"), torch.empty(T, n, device="cuda")
    q8 = ops.Q8Buffers(T * n, "cuda", xh="bf16")
    ops.gpu_gemma_ffn_post(dev(x), dev(mlp), dev(down), dev(wts), dev(ids), dev(es) if scaled else None, n_used, dev(w1),
                           dev(w2), dev(w_post), ds, x_out, dev(w_next), y, n, T, 1e-6, q8=q8)
    torch.cuda.synchronize()
    wx, wy = oracle.gemma_ffn_post(x, mlp, down, wts, ids, es if scaled else None, w1, w2, w_post, scale, w_next, 1e-6)
    assert np.array_equal(host(x_out).view(np.uint32), wx.view(np.uint32))
    assert np.array_equal(host(y).view(np.uint32), wy.view(np.uint32))
    want = oracle.quantize_q8(host(y), xh="bf16")
    for k in ("q0", "d0", "s0", "qK", "dK", "bsK"):
        assert np.array_equal(host(getattr(q8, k)).view(want[k].dtype), want[k]), k
    # the unfused branch of the reference (src/qwen_model.cpp:1364-1382): combine, add_normed x3, the plain norm
    c, h, xo2, y2 = (torch.empty(T, n, device="cuda") for _ in range(4))
    ops.gpu_moe_combine(dev(down), dev(wts), None, None, c, n_used, n, T, dev(ids) if scaled else None,
                        dev(es) if scaled else None)
    ops.gpu_add_rmsnorm(dev(mlp), None, None, dev(w1), h, n, T, 1e-6)
    ops.gpu_add_normed(h, c, dev(w2), None, h, n, T, 1e-6)
    ops.gpu_add_normed(dev(x), h, dev(w_post), ds, xo2, n, T, 1e-6)
    ops.gpu_add_rmsnorm(xo2, None, None, dev(w_next), y2, n, T, 1e-6)
    torch.cuda.synchronize()
    assert max_rel_rows(host(xo2), host(x_out)) <= 1e-6 and max_rel_rows(host(y2), host(y)) <= 1e-6
    with pytest.raises(ops.LayerOpError):
        xx = dev(x)
        ops.gpu_gemma_ffn_post(xx, dev(mlp), dev(down), dev(wts), dev(ids), None, n_used, dev(w1), dev(w2), dev(w_post),
                               None, xx, dev(w_next), y, n, T, 1e-6)
