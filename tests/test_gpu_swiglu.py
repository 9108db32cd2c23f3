"""CUDA SwiGLU against the CPU oracle through the C ABI. fp32: worst row of max|d|/max|ref| <= 1e-5 (rows of the FFN
width). bf16: within 1 bf16 ulp of the oracle."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import bf16_ulp_dist, dev, host, max_rel_rows

pytestmark = pytest.mark.gpu


def test_c1_fp32(ops, oracle):
    """Qwen3-0.6B shape: two 2427 x 3072 inputs ~ N(0,1)."""
    T, FF = 2427, 3072
    g = synth.normal(0, "c1.ffg", 0, T * FF)
    u = synth.normal(0, "c1.ffu", 0, T * FF)
    want = oracle.swiglu(g, u)
    dg, du = dev(g), dev(u)
    out = torch.full_like(dg, float("nan"))
    ops.gpu_swiglu(dg, du, out, T * FF)
    torch.cuda.synchronize()
    got = host(out)
    assert max_rel_rows(got.reshape(T, FF), want.reshape(T, FF)) <= 1e-5
    # per value it is much tighter than the row metric asks: a few ulp
    assert np.abs(got - want).max() <= 4e-7 * np.abs(want).max() + 1e-12 or \
        (np.abs(got - want) / np.maximum(np.abs(want), 1e-30)).max() < 1e-5


@pytest.mark.parametrize("n", [1, 3, 4, 5, 255, 1024, 4099, 1 << 20, (1 << 20) + 7])
def test_sizes_and_tails_fp32(ops, oracle, n):
    g = synth.normal(4, "t.g", 0, n) * 3
    u = synth.normal(4, "t.u", 0, n)
    want = oracle.swiglu(g, u)
    out = torch.full((n + 8,), 7.0, device="cuda")
    ops.gpu_swiglu(dev(g), dev(u), out, n)
    torch.cuda.synchronize()
    got = host(out)
    assert (got[n:] == 7).all()
    assert max_rel_rows(got[:n], want) <= 1e-5


def test_unaligned_pointers(ops, oracle):
    n = 10007
    g = synth.normal(5, "u.g", 0, n + 3)
    u = synth.normal(5, "u.u", 0, n + 3)
    dg, du = dev(g), dev(u)
    out = torch.zeros(n + 3, device="cuda")
    ops.gpu_swiglu(dg[1:], du[3:], out[1:], n)   # 4-byte aligned only
    torch.cuda.synchronize()
    assert max_rel_rows(host(out)[1:n + 1], oracle.swiglu(g[1:n + 1], u[3:n + 3])) <= 1e-5
    gb = oracle.f32_to_bf16(g)
    ub = oracle.f32_to_bf16(u)
    outb = torch.zeros(n + 3, device="cuda", dtype=torch.bfloat16)
    ops.gpu_swiglu(dev(gb, torch.bfloat16)[1:], dev(ub, torch.bfloat16)[2:], outb[1:], n)
    torch.cuda.synchronize()
    assert bf16_ulp_dist(host(outb)[1:n + 1], oracle.swiglu_bf16(gb[1:n + 1], ub[2:n + 2])).max() <= 1


def test_extreme_gates(ops, oracle):
    """Large |g|: exp overflows to infinity for very negative gates and the result is a signed zero or a tiny value;
    the fast 16-bit path must keep those instead of flushing."""
    g = np.array([-104, -100, -89, -88.5, -88, -87, -50, -20, -10, -1, -1e-3, -0.0, 0.0, 1e-3, 1, 10, 20, 50, 88, 89,
                  100, 1e4, -1e4, 3e38, -3e38], dtype=np.float32)
    g = np.concatenate([g, np.linspace(-95, 95, 4071, dtype=np.float32)])
    u = np.where(np.arange(g.size) % 2 == 0, 1.5, -0.75).astype(np.float32)
    want = oracle.swiglu(g, u)
    out = torch.zeros(g.size, device="cuda")
    ops.gpu_swiglu(dev(g), dev(u), out, g.size)
    torch.cuda.synchronize()
    got = host(out)
    assert np.isfinite(got).all()
    rel = np.abs(got - want) / np.maximum(np.abs(want), 1e-37)
    assert rel.max() < 1e-5
    gb, ub = oracle.f32_to_bf16(g), oracle.f32_to_bf16(u)
    outb = torch.zeros(g.size, device="cuda", dtype=torch.bfloat16)
    ops.gpu_swiglu(dev(gb, torch.bfloat16), dev(ub, torch.bfloat16), outb, g.size)
    torch.cuda.synchronize()
    assert bf16_ulp_dist(host(outb), oracle.swiglu_bf16(gb, ub)).max() <= 1


def test_c3_c4_shapes_bf16(ops, oracle):
    """Dense FFN rows (intermediate 9216) and expert-grouped rows (512 wide, rows sorted by expert id): the map is
    flat, so grouped rows are the same values in another order."""
    for rows, width, name in ((512, 9216, "c3"), (4096, 512, "c4")):
        g = oracle.f32_to_bf16(synth.normal(0, name + ".g", 0, rows * width))
        u = oracle.f32_to_bf16(synth.normal(0, name + ".u", 0, rows * width))
        want = oracle.swiglu_bf16(g, u)
        out = torch.zeros(rows * width, device="cuda", dtype=torch.bfloat16)
        ops.gpu_swiglu(dev(g, torch.bfloat16), dev(u, torch.bfloat16), out, rows * width)
        torch.cuda.synchronize()
        got = host(out)
        d = bf16_ulp_dist(got, want)
        assert d.max() <= 1
        assert (d != 0).mean() < 1e-3          # the fast path lands on the same bf16 value almost always
        if name == "c4":                        # group the rows by expert: same rows, permuted
            ids, order = synth.moe_routing(0, "c4.route", rows // 8, 256, 8)
            perm = torch.from_numpy(order).cuda()
            gg = dev(g, torch.bfloat16).view(rows, width)[perm].contiguous()
            uu = dev(u, torch.bfloat16).view(rows, width)[perm].contiguous()
            out2 = torch.zeros(rows, width, device="cuda", dtype=torch.bfloat16)
            ops.gpu_swiglu(gg, uu, out2, rows * width)
            assert torch.equal(out2, out.view(rows, width)[perm])


def test_fused_gate_up_rows(ops, oracle):
    """gpu_swiglu_rows on rows laid out [gate | up] (stride 2 h), vector and scalar paths."""
    for rows, h, dt in ((300, 512, torch.float32), (300, 512, torch.bfloat16), (17, 100, torch.float32), (5, 37, torch.bfloat16)):
        gu = synth.normal(6, f"gu{h}", 0, rows * 2 * h).reshape(rows, 2 * h)
        if dt == torch.float32:
            want = oracle.swiglu(gu[:, :h], gu[:, h:])
            d = dev(gu)
        else:
            b = oracle.f32_to_bf16(gu).reshape(rows, 2 * h)
            want = oracle.swiglu_bf16(b[:, :h], b[:, h:])
            d = dev(b, dt)
        out = torch.zeros(rows, h, device="cuda", dtype=dt)
        ops.gpu_swiglu_rows(d, d[:, h:], out, rows, h, 2 * h, 2 * h)
        torch.cuda.synchronize()
        if dt == torch.float32:
            assert max_rel_rows(host(out), want) <= 1e-5
        else:
            assert bf16_ulp_dist(host(out), want).max() <= 1


def test_q8_side_outputs(ops, oracle):
    n = 8 * 256 + 96   # whole Q8_0 blocks, a partial Q8_K block at the end (src/gpu_ops.h:27-29)
    g = synth.normal(7, "sq.g", 0, n)
    u = synth.normal(7, "sq.u", 0, n)
    q8 = ops.Q8Buffers(9 * 256, "cuda", xh="bf16")
    out = torch.zeros(n, device="cuda")
    ops.gpu_swiglu(dev(g), dev(u), out, n, q8=q8)
    torch.cuda.synchronize()
    y = host(out)
    full = 8 * 256
    want = oracle.quantize_q8(y[:full], xh="bf16")
    for k, per in (("q0", 1), ("d0", 32), ("s0", 32), ("qK", 1), ("dK", 256), ("bsK", 16)):
        assert np.array_equal(host(getattr(q8, k))[: full // per].view(want[k].dtype), want[k]), k
    assert np.array_equal(host(q8.xh).view(np.uint16)[:n], oracle.f32_to_bf16(y))
    tail = oracle.quantize_q8(np.concatenate([y[full:], np.zeros(160, np.float32)]))
    assert np.array_equal(host(q8.q0)[full:n], tail["q0"][:96])
    assert np.array_equal(host(q8.d0)[full // 32: n // 32], tail["d0"][:3])
    with pytest.raises(ops.LayerOpError) as e:
        ops.gpu_swiglu(dev(g), dev(u), out, n - 1, q8=q8)      # n % 32 != 0 with q8 (src/gpu_ops.cpp:82)
    assert e.value.code == 1


@pytest.mark.parametrize("n", [256 * 1000 + 64, 4 * 1024 * 33, 1056])
def test_16_bit_side_copy_comes_from_the_swiglu_kernel_itself(ops, oracle, n):
    """Only the 16-bit copy wanted (src/q8_device.h:58): one launch writes out and out rounded to bf16 / fp16."""
    g, u = synth.normal(7, "sx.g", 0, n), synth.normal(7, "sx.u", 0, n)
    dg, du = dev(g), dev(u)
    for kind in ("bf16", "f16"):
        conv = oracle.f32_to_bf16 if kind == "bf16" else oracle.f32_to_f16
        q8 = ops.Q8Buffers((n + 255) // 256 * 256, "cuda", xh=kind, int8=False)
        out, plain = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        before = ops.launch_count()
        ops.gpu_swiglu(dg, du, out, n, q8=q8)
        assert ops.launch_count() - before == 1
        ops.gpu_swiglu(dg, du, plain, n)
        torch.cuda.synchronize()
        assert np.array_equal(host(out).view(np.uint32), host(plain).view(np.uint32))
        assert np.array_equal(host(q8.xh).view(np.uint16)[:n], conv(host(out)).reshape(-1))
        assert not host(q8.xh)[n:].any()
