"""The kernels the reference looks up by name ("add_rmsnorm", "add_rmsnorm_rows", "swiglu", "rmsnorm",
"rope_rotate_half"), loaded from rocm_hip_b200/gpu_ops.fatbin with the driver's module API and launched with the
reference's own grid / block shapes and argument lists (src/gpu_ops.cpp:66-86, tests/layernorm_verify.cpp:93-97,
tests/rope_verify.cpp:111-114), checked against the CPU oracle."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import dev, host, max_rel_rows

pytestmark = pytest.mark.gpu
FATBIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "rocm_hip_b200", "gpu_ops.fatbin")


class Q8Out(C.Structure):   # src/q8_device.h:22-31
    _fields_ = [("q0", C.c_void_p), ("d0", C.c_void_p), ("qK", C.c_void_p), ("dK", C.c_void_p), ("bsK", C.c_void_p),
                ("s0", C.c_void_p), ("xh", C.c_void_p), ("xh_bf16", C.c_int)]


@pytest.fixture(scope="module")
def module(ops):
    from cuda.bindings import driver as drv
    torch.zeros(1, device="cuda")   # make sure the primary context is current
    err, mod = drv.cuModuleLoadData(open(FATBIN, "rb").read())
    assert err == drv.CUresult.CUDA_SUCCESS, err

    def launch(name, grid, block, *args):
        err, fn = drv.cuModuleGetFunction(mod, name.encode())
        assert err == drv.CUresult.CUDA_SUCCESS, (name, err)
        ptrs = (C.c_void_p * len(args))(*[C.addressof(a) for a in args])
        (err,) = drv.cuLaunchKernel(fn, grid[0], grid[1], 1, block, 1, 1, 0, torch.cuda.current_stream().cuda_stream,
                                    C.addressof(ptrs), 0)
        assert err == drv.CUresult.CUDA_SUCCESS, (name, err)
        torch.cuda.synchronize()

    yield launch
    drv.cuModuleUnload(mod)


def p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def test_add_rmsnorm_both_shapes(module, oracle, ops):
    for T, n in ((1, 1024), (5, 2560), (3, 1000), (4, 5120)):
        x = synth.normal(0, "nk.x", 0, T * n).reshape(T, n)
        a = synth.normal(0, "nk.a", 0, T * n).reshape(T, n)
        w = synth.normal(0, "nk.w", 0, n, 1.0, 0.1)
        for add in (None, a):
            wxo, want = oracle.add_rmsnorm(x, add, w, 1e-6)
            names = ["add_rmsnorm"] + (["add_rmsnorm_rows"] if n % 256 == 0 else [])
            for name in names:
                dx, da, dw = dev(x), dev(add), dev(w)
                xo, y = torch.zeros_like(dx), torch.zeros_like(dx)
                grid = ((n + 255) // 256, T) if name == "add_rmsnorm" else (T, 1)
                module(name, grid, 256, p(dx), p(da), p(xo), p(dw), p(y), C.c_int(n), C.c_float(1e-6), Q8Out())
                assert max_rel_rows(host(y), want) <= 1e-5
                assert np.array_equal(host(y).view(np.uint32), want.view(np.uint32))   # bit for bit, in fact
                if add is not None:
                    assert np.array_equal(host(xo).view(np.uint32), wxo.view(np.uint32))
    # with the side outputs, as the launcher passes them when q8 is set (n % 256 == 0)
    T, n = 3, 1024
    x = synth.normal(1, "nk.x", 0, T * n).reshape(T, n)
    dx = dev(x)
    y = torch.zeros_like(dx)
    q8 = ops.Q8Buffers(T * n, "cuda", xh="bf16")
    o = Q8Out(q8.q0.data_ptr(), q8.d0.data_ptr(), q8.qK.data_ptr(), q8.dK.data_ptr(), q8.bsK.data_ptr(),
              q8.s0.data_ptr(), q8.xh.data_ptr(), 1)
    module("add_rmsnorm_rows", (T, 1), 256, p(dx), p(None), p(dx), p(None), p(y), C.c_int(n), C.c_float(1e-6), o)
    want = oracle.quantize_q8(host(y), xh="bf16")
    for k in ("q0", "d0", "s0", "qK", "dK", "bsK"):
        assert np.array_equal(host(getattr(q8, k)).view(want[k].dtype), want[k]), k
    assert np.array_equal(host(q8.xh).view(np.uint16), want["xh"])


def test_swiglu(module, oracle):
    n = 10000
    g, u = synth.normal(0, "nk.g", 0, n) * 3, synth.normal(0, "nk.u", 0, n)
    out = torch.zeros(n, device="cuda")
    dg, du = dev(g), dev(u)   # (kept alive: a raw pointer does not hold the tensor)
    module("swiglu", ((n + 255) // 256, 1), 256, p(dg), p(du), p(out), C.c_int(n), Q8Out())
    assert max_rel_rows(host(out), oracle.swiglu(g, u)) <= 1e-5


def test_fp16_component_kernels_as_the_reference_tests_launch_them(module, oracle):
    """tests/layernorm_verify.cpp and tests/rope_verify.cpp: grid = rows, block = 32, their seeds, shapes and rule."""
    for tokens, embd in ((8, 17), (32, 64), (5, 4096), (1, 96), (7, 48)):
        rng = oracle.Lcg(7)
        x = np.array([rng.rnd(-3.0, 3.0) for _ in range(tokens * embd)], dtype=np.float32)
        gam = np.array([rng.rnd(0.5, 1.5) for _ in range(embd)], dtype=np.float32)
        xh, gh = oracle.f32_to_f16(x).reshape(tokens, embd), oracle.f32_to_f16(gam)
        want = oracle.rmsnorm_f16(xh, gh, 1e-5)
        dx, dg = dev(xh, torch.float16), dev(gh, torch.float16)
        dy = torch.zeros_like(dx)
        module("rmsnorm", (tokens, 1), 32, p(dx), p(dg), p(dy), C.c_int(tokens), C.c_int(embd), C.c_float(1e-5))
        g, r = oracle.f16_to_f32(host(dy)), oracle.f16_to_f32(want)
        assert not (np.abs(g - r) > 0.01 * np.maximum(np.abs(g), np.abs(r)) + 1e-4).any()
        assert np.abs(host(dy).astype(np.int32) - want.astype(np.int32)).max() <= 1
    state, positions = 99, []
    for _ in range(64):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        positions.append(1 + (state >> 8) % 4096)
    positions = np.array(positions, dtype=np.int32)
    for rows, dim in ((16, 16), (5, 32), (64, 128)):
        rng = oracle.Lcg(13)
        x = oracle.f32_to_f16(np.array([rng.rnd(-3.0, 3.0) for _ in range(rows * dim)], dtype=np.float32)).reshape(rows, dim)
        c, s = oracle.rope_tables(positions[:rows], dim, 10000.0)
        want = oracle.rope_rotate_half_f16(x, c, s)
        dx = dev(x, torch.float16)
        dy = torch.zeros_like(dx)
        dc, ds = dev(c), dev(s)
        module("rope_rotate_half", (rows, 1), 32, p(dx), p(dc), p(ds), p(dy), C.c_int(rows), C.c_int(dim // 2))
        assert np.array_equal(host(dy), want)
