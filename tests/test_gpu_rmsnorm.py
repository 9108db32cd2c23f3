"""CUDA residual-add + RMSNorm against the CPU oracle, through the C ABI (rocm_hip_b200.ops -> libb200_layer_ops.so).
fp32: worst row of max|d|/max|ref| <= 1e-5. bf16: every value within 1 bf16 ulp of the oracle. x_out: bit-exact."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import bf16_ulp_dist, dev, host, max_rel_rows

pytestmark = pytest.mark.gpu
TOL32 = 1e-5


def run_f32(ops, x, add, w, eps, inplace=False):
    T, n = x.shape
    dx, da, dw = dev(x), dev(add), dev(w)
    xo = torch.full_like(dx, float("nan")) if add is not None else None
    y = dx if inplace else torch.full_like(dx, float("nan"))
    ops.gpu_add_rmsnorm(dx, da, xo if xo is not None else dx, dw, y, n, T, eps)
    torch.cuda.synchronize()
    return (host(xo) if xo is not None else None), host(y)


def run_bf16(ops, x, add, w, eps):
    T, n = x.shape
    dx, da, dw = dev(x, torch.bfloat16), dev(add, torch.bfloat16), dev(w)
    xo = torch.zeros_like(dx) if add is not None else None
    y = torch.zeros_like(dx)
    ops.gpu_add_rmsnorm(dx, da, xo if xo is not None else dx, dw, y, n, T, eps)
    torch.cuda.synchronize()
    return (host(xo) if xo is not None else None), host(y)


def test_c1_model_norm_fp32(ops, oracle):
    """Qwen3-0.6B shape: 2,427 tokens x hidden 1024, eps 1e-6, x ~ N(0,1), w ~ N(1,0.1); plain and with the residual."""
    T, n = 2427, 1024
    x = synth.normal(0, "c1.x", 0, T * n).reshape(T, n)
    a = synth.normal(0, "c1.add", 0, T * n).reshape(T, n)
    w = synth.normal(0, "c1.w", 0, n, 1.0, 0.1)
    _, want = oracle.add_rmsnorm(x, None, w, 1e-6)
    _, got = run_f32(ops, x, None, w, 1e-6)
    assert max_rel_rows(got, want) <= TOL32
    _, got_ip = run_f32(ops, x, None, w, 1e-6, inplace=True)   # y == x_in is legal without add
    assert np.array_equal(got_ip.view(np.uint32), got.view(np.uint32))
    wxo, want = oracle.add_rmsnorm(x, a, w, 1e-6)
    gxo, got = run_f32(ops, x, a, w, 1e-6)
    assert np.array_equal(gxo.view(np.uint32), wxo.view(np.uint32))
    assert max_rel_rows(got, want) <= TOL32


def test_c1_per_head_norm_fp32(ops, oracle):
    """q/k norm as a plain row norm: 2,427 x (16 + 8) head rows of 128."""
    R, n = 2427 * 24, 128
    x = synth.normal(0, "c1.qk", 0, R * n).reshape(R, n)
    w = synth.normal(0, "c1.qkw", 0, n, 1.0, 0.1)
    _, want = oracle.add_rmsnorm(x, None, w, 1e-6)
    _, got = run_f32(ops, x, None, w, 1e-6)
    assert max_rel_rows(got, want) <= TOL32


@pytest.mark.parametrize("n", [4, 17, 48, 96, 128, 256, 1000, 1024, 2048, 2560, 4096, 5120, 8192, 10240, 33000])
@pytest.mark.parametrize("T", [1, 7])
def test_shapes_fp32(ops, oracle, n, T):
    """Every launch shape: lane groups, one CTA per row, wide rows, and widths that fall back to scalar accesses
    (the reference's own sweep widths 17, 48, 96 among them); gamma NULL too."""
    x = synth.normal(1, f"s.x{n}", 0, T * n).reshape(T, n)
    a = synth.normal(1, f"s.a{n}", 0, T * n).reshape(T, n)
    w = synth.normal(1, f"s.w{n}", 0, n, 1.0, 0.1)
    for add, ww in ((None, w), (a, w), (a, None)):
        wxo, want = oracle.add_rmsnorm(x, add, ww, 1e-5)
        gxo, got = run_f32(ops, x, add, ww, 1e-5)
        assert max_rel_rows(got, want) <= TOL32
        if add is not None:
            assert np.array_equal(gxo.view(np.uint32), wxo.view(np.uint32))


@pytest.mark.parametrize("n", [8, 24, 128, 256, 1000, 1024, 2048, 2560, 5120, 16384])
@pytest.mark.parametrize("T", [1, 64, 333])
def test_shapes_bf16(ops, oracle, n, T):
    x = oracle.f32_to_bf16(synth.normal(2, f"b.x{n}", 0, T * n)).reshape(T, n)
    a = oracle.f32_to_bf16(synth.normal(2, f"b.a{n}", 0, T * n)).reshape(T, n)
    w = synth.normal(2, f"b.w{n}", 0, n, 1.0, 0.1)
    for add in (None, a):
        wxo, want = oracle.add_rmsnorm_bf16(x, add, w, 1e-6)
        gxo, got = run_bf16(ops, x, add, w, 1e-6)
        assert bf16_ulp_dist(got, want).max() <= 1
        if add is not None:
            assert np.array_equal(gxo, wxo)


def test_row_bits_do_not_depend_on_batch(ops):
    """A row gives the same bits alone, in a batch, and at another place of a batch (what row sharding relies on)."""
    for n, dt in ((1024, torch.float32), (5120, torch.bfloat16), (128, torch.bfloat16), (2560, torch.float32)):
        T = 301
        g = torch.Generator(device="cuda").manual_seed(5)
        x = torch.randn(T, n, device="cuda", generator=g).to(dt)
        a = torch.randn(T, n, device="cuda", generator=g).to(dt)
        w = (1 + 0.1 * torch.randn(n, device="cuda", generator=g)).float()
        xo, y = torch.empty_like(x), torch.empty_like(x)
        ops.gpu_add_rmsnorm(x, a, xo, w, y, n, T, 1e-6)
        for lo, hi in ((0, 1), (300, 301), (17, 150), (150, 301)):
            xs, as_ = x[lo:hi].contiguous(), a[lo:hi].contiguous()
            xo2, y2 = torch.empty_like(xs), torch.empty_like(xs)
            ops.gpu_add_rmsnorm(xs, as_, xo2, w, y2, n, hi - lo, 1e-6)
            assert torch.equal(y2.view(torch.int16 if dt != torch.float32 else torch.int32),
                               y[lo:hi].view(torch.int16 if dt != torch.float32 else torch.int32))
            assert torch.equal(xo2, xo[lo:hi])


def test_guard_bands_untouched(ops):
    """Nothing is written outside the T x n outputs (the reference has no sanitizer either: canaries stand in)."""
    for n, T, dt in ((1000, 3, torch.float32), (1024, 5, torch.float32), (5120, 3, torch.bfloat16), (24, 9, torch.bfloat16)):
        pad = 64
        buf_y = torch.full((T * n + 2 * pad,), 7.0, device="cuda", dtype=dt)
        buf_o = torch.full((T * n + 2 * pad,), 7.0, device="cuda", dtype=dt)
        x = torch.randn(T, n, device="cuda").to(dt)
        a = torch.randn(T, n, device="cuda").to(dt)
        y = buf_y[pad:pad + T * n].view(T, n)
        xo = buf_o[pad:pad + T * n].view(T, n)
        ops.gpu_add_rmsnorm(x, a, xo, None, y, n, T, 1e-6)
        torch.cuda.synchronize()
        for b in (buf_y, buf_o):
            assert (b[:pad] == 7).all() and (b[-pad:] == 7).all()
        assert not (y == 7).all()


def test_fp16_component_sweep(ops, oracle):
    """The reference's layernorm_verify sweep (tests/layernorm_verify.cpp:64-76,139) through gpu_rmsnorm_f16, judged
    by that test's own rule and, tighter, to one fp16 ulp of the restated CPU reference."""
    for tokens, embd in ((8, 17), (32, 64), (5, 4096), (1, 96), (7, 48)):
        rng = oracle.Lcg(7)
        x = np.array([rng.rnd(-3.0, 3.0) for _ in range(tokens * embd)], dtype=np.float32)
        gam = np.array([rng.rnd(0.5, 1.5) for _ in range(embd)], dtype=np.float32)
        xh, gh = oracle.f32_to_f16(x).reshape(tokens, embd), oracle.f32_to_f16(gam)
        for gamma in (gh, None):
            want = oracle.rmsnorm_f16(xh, gamma, 1e-5)
            dx = dev(xh, torch.float16)
            dy = torch.zeros_like(dx)
            ops.gpu_rmsnorm_f16(dx, dev(gamma, torch.float16), dy, tokens, embd, 1e-5)
            torch.cuda.synchronize()
            g, r = oracle.f16_to_f32(host(dy)), oracle.f16_to_f32(want)
            assert not (np.abs(g - r) > 0.01 * np.maximum(np.abs(g), np.abs(r)) + 1e-4).any()
            assert np.abs(host(dy).astype(np.int32) - want.astype(np.int32)).max() <= 1


def test_q8_side_outputs(ops, oracle):
    """gpu_add_rmsnorm with a qmatvec_q8: the int8 / bf16 copies are exactly the reference's quantisation rules
    (src/q8_device.h:54-104) applied to the y the kernel wrote."""
    T, n = 9, 1024
    x = synth.normal(3, "q8.x", 0, T * n).reshape(T, n)
    w = synth.normal(3, "q8.w", 0, n, 1.0, 0.1)
    dx, dw = dev(x), dev(w)
    y = torch.empty_like(dx)
    for xh in ("bf16", "f16"):
        q8 = ops.Q8Buffers(T * n, "cuda", xh=xh)
        ops.gpu_add_rmsnorm(dx, None, dx, dw, y, n, T, 1e-6, q8=q8)
        torch.cuda.synchronize()
        want = oracle.quantize_q8(host(y), xh=xh)
        for k in ("q0", "d0", "s0", "qK", "dK", "bsK"):
            assert np.array_equal(host(getattr(q8, k)).view(want[k].dtype), want[k]), k
        assert np.array_equal(host(q8.xh).view(np.uint16), want["xh"])
    # the reference's argument rules (src/gpu_ops.cpp:69): n % 256 and max_k
    small = ops.Q8Buffers(256, "cuda")
    with pytest.raises(ops.LayerOpError) as e:
        ops.gpu_add_rmsnorm(dx, None, dx, dw, y, n, T, 1e-6, q8=small)
    assert e.value.code == 1


@pytest.mark.parametrize("n,T", [(4096, 33), (1024, 300), (2560, 17)])
def test_16_bit_side_copy_comes_from_the_norm_kernel_itself(ops, oracle, n, T):
    """A qmatvec_q8 that asks only for the 16-bit copy (src/q8_device.h:58): xh = y rounded to bf16 / fp16, written by
    the one norm launch when the row shape takes the trimmed kernel; with the int8 formats also wanted, or without
    gammas, one more launch; the bits are the same either way."""
    x = synth.normal(3, "xh.x", 0, T * n).reshape(T, n)
    a = synth.normal(3, "xh.a", 0, T * n).reshape(T, n)
    w = synth.normal(3, "xh.w", 0, n, 1.0, 0.1)
    dx, da, dw = dev(x), dev(a), dev(w)
    for kind in ("bf16", "f16"):
        conv = oracle.f32_to_bf16 if kind == "bf16" else oracle.f32_to_f16
        for add in (None, da):
            q8 = ops.Q8Buffers(T * n, "cuda", xh=kind, int8=False)
            y, xo, y_plain = torch.empty_like(dx), torch.empty_like(dx), torch.empty_like(dx)
            before = ops.launch_count()
            ops.gpu_add_rmsnorm(dx, add, xo, dw, y, n, T, 1e-6, q8=q8)
            assert ops.launch_count() - before == 1
            ops.gpu_add_rmsnorm(dx, add, xo, dw, y_plain, n, T, 1e-6)
            torch.cuda.synchronize()
            assert np.array_equal(host(y).view(np.uint32), host(y_plain).view(np.uint32))
            assert np.array_equal(host(q8.xh).view(np.uint16), conv(host(y)).reshape(-1))
        q8 = ops.Q8Buffers(T * n, "cuda", xh=kind, int8=False)
        y = torch.empty_like(dx)
        before = ops.launch_count()
        ops.gpu_add_rmsnorm(dx, None, dx, None, y, n, T, 1e-6, q8=q8)       # no gammas: the general kernel + side kernel
        torch.cuda.synchronize()
        assert ops.launch_count() - before == 2
        assert np.array_equal(host(q8.xh).view(np.uint16), conv(host(y)).reshape(-1))


def test_argument_errors(ops):
    """src/gpu_ops.cpp:68-70: not initialised -> cudaErrorInvalidDeviceFunction (98); T <= 0 or add with
    x_out == x_in -> cudaErrorInvalidValue (1). Nothing is launched in either case."""
    x = torch.randn(4, 256, device="cuda")
    y = torch.empty_like(x)
    before = ops.launch_count()
    with pytest.raises(ops.LayerOpError) as e:
        ops.gpu_add_rmsnorm(x, x, x, None, y, 256, 4, 1e-6)
    assert e.value.code == 1
    with pytest.raises(ops.LayerOpError) as e:
        ops.gpu_add_rmsnorm(x, None, x, None, y, 256, 0, 1e-6)
    assert e.value.code == 1
    ops.gpu_ops_free()
    try:
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_add_rmsnorm(x, None, x, None, y, 256, 4, 1e-6)
        assert e.value.code == 98
    finally:
        assert ops.gpu_ops_init("gpu_ops.co") == 0
    assert ops.launch_count() == before
    assert ops.gpu_ops_init("gpu_ops.co") == 0  # idempotent
