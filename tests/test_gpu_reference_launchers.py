"""The reference's own launcher source (src/gpu_ops.cpp) and module loader (src/kernel_loader.cpp), compiled UNCHANGED
against the hip/ shim headers into oracle/_ref/libref_gpu_ops.so (oracle/Makefile, target ref_programs), driving this
library's kernels: INFERENCE_KERNEL_DIR points at a directory holding rocm_hip_b200/gpu_ops.fatbin as gpu_ops.co, the
reference's gpu_ops_init finds all 23 kernels it asks for by name (src/gpu_ops.cpp:26-48), and every one of its
launchers then gives the results of this library's native launcher of the same name on the same inputs (identical up
to the summation order inside a row reduction: compared at 1e-6 of the row maximum; integer outputs exactly)."""
import ctypes as C
import os
import shutil

import numpy as np
import pytest
import torch

from rocm_hip_b200 import _lib
from util import max_rel_rows

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_gpu_ops.so")
NAMES = ["gpu_add_rmsnorm", "gpu_swiglu", "gpu_moe_router", "gpu_moe_combine", "gpu_moe_combine_scaled", "gpu_moe_group",
         "gpu_add_normed", "gpu_gemma_attn_post", "gpu_gemma_ffn_post", "gpu_geglu", "gpu_softcap", "gpu_hc_norm",
         "gpu_hc_lowrank", "gpu_hc_mix", "gpu_ple_gate", "gpu_ple_conv", "gpu_mtp_concat", "gpu_mamba_conv", "gpu_mamba_scan",
         "gpu_mamba_gnorm", "gpu_moe_router_sigmoid", "gpu_relu2"]


@pytest.fixture(scope="module")
def both(ops, tmp_path_factory):
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libref_gpu_ops.so was not built (the reference's source tree was absent at build time)")
    d = tmp_path_factory.mktemp("kernels")
    shutil.copy(os.path.join(ROOT, "rocm_hip_b200", "gpu_ops.fatbin"), d / "gpu_ops.co")
    os.environ["INFERENCE_KERNEL_DIR"] = str(d)
    ref = C.CDLL(REF_LIB)
    ref.gpu_ops_init.restype, ref.gpu_ops_init.argtypes = C.c_int, [C.c_char_p]
    for n in NAMES:
        getattr(ref, n).restype, getattr(ref, n).argtypes = _lib.SIGNATURES[n]
    assert ref.gpu_ops_init(b"gpu_ops.co") == 0, "the reference's gpu_ops_init did not find its kernels in the module image"
    yield ref, _lib.load()
    ref.gpu_ops_free()
    del os.environ["INFERENCE_KERNEL_DIR"]


P = lambda t: None if t is None else C.c_void_p(t.data_ptr())
R = lambda *s: torch.randn(*s, device="cuda")
Z = lambda *s: torch.zeros(*s, device="cuda")
ST = C.c_void_p(0)


def run_both(both, name, make_args, outputs, exact=False):
    """Calls launcher `name` of the reference build and of this library with fresh argument lists from make_args()
    (which returns (args, output tensors)) and compares the outputs."""
    ref, mine = both
    res = []
    for lib in (ref, mine):
        torch.manual_seed(1234)
        args, outs = make_args()
        code = getattr(lib, name)(*args)
        torch.cuda.synchronize()
        assert code == 0, (name, code)
        res.append([o.clone() for o in outs])
    for a, b in zip(*res):
        if exact or a.dtype != torch.float32:
            assert torch.equal(a, b), name
        else:
            an, bn = a.cpu().numpy(), b.cpu().numpy()
            assert max_rel_rows(an.reshape(an.shape[0], -1), bn.reshape(bn.shape[0], -1)) <= 1e-6, name


def q8_struct(K, keep):
    bufs = dict(q0=torch.zeros(K, dtype=torch.int8, device="cuda"), d0=Z(K // 32), qK=torch.zeros(K, dtype=torch.int8, device="cuda"),
                dK=Z(K // 256), bsK=torch.zeros(K // 16, dtype=torch.int32, device="cuda"),
                s0=torch.zeros(K // 32, dtype=torch.int32, device="cuda"), xh=torch.zeros(K, dtype=torch.int16, device="cuda"))
    keep.append(bufs)
    g = lambda k: bufs[k].data_ptr()
    return _lib.qmatvec_q8(g("q0"), g("d0"), g("qK"), g("dK"), g("bsK"), g("s0"), K, g("xh"), 1), bufs


def test_norms_and_activations(both):
    keep = []
    T, n = 9, 1024

    def rms(add, q8):
        def mk():
            x, a, w = R(T, n), R(T, n), 1 + 0.1 * R(n)
            xo, y = Z(T, n), Z(T, n)
            s, bufs = q8_struct(T * n, keep) if q8 else (None, {})
            keep.extend([x, a, w])
            return [P(x), P(a) if add else None, P(xo), P(w), P(y), n, T, 1e-6, C.byref(s) if q8 else None, ST], \
                [y, xo] + [bufs[k] for k in ("q0", "qK", "xh")] if q8 else [y, xo]
        return mk
    for add in (False, True):
        for q8 in (False, True):
            run_both(both, "gpu_add_rmsnorm", rms(add, q8), None)

    def swiglu():
        g, u, o = R(T * n), R(T * n), Z(T * n)
        s, bufs = q8_struct(T * n, keep)
        keep.extend([g, u])
        return [P(g), P(u), P(o), T * n, C.byref(s), ST], [o.view(T, n), bufs["q0"], bufs["xh"]]
    run_both(both, "gpu_swiglu", swiglu, None)

    def add_normed():
        b, a, w, sc, o = R(T, n), R(T, n), 1 + 0.1 * R(n), torch.tensor([0.7], device="cuda"), Z(T, n)
        keep.extend([b, a, w, sc])
        return [P(b), P(a), P(w), P(sc), P(o), n, T, 1e-6, ST], [o]
    run_both(both, "gpu_add_normed", add_normed, None)

    def attn_post():
        x, a, wa, w1, w2 = R(T, n), R(T, n), 1 + 0.1 * R(n), 1 + 0.1 * R(n), 1 + 0.1 * R(n)
        xo, y1, y2 = Z(T, n), Z(T, n), Z(T, n)
        s, bufs = q8_struct(T * n, keep)
        keep.extend([x, a, wa, w1, w2])
        return [P(x), P(a), P(wa), P(xo), P(w1), P(y1), C.byref(s), P(w2), P(y2), n, T, 1e-6, ST], [xo, y1, y2, bufs["qK"]]
    run_both(both, "gpu_gemma_attn_post", attn_post, None)

    def geglu():
        gu, o = R(T, 2 * n), Z(T, n)
        keep.append(gu)
        return [P(gu), C.c_void_p(gu.data_ptr() + 4 * n), P(o), T, n, 2 * n, 2 * n, None, ST], [o]
    run_both(both, "gpu_geglu", geglu, None)

    def relu2():
        x, o = R(T, n + 8), Z(T, n)
        keep.append(x)
        return [P(x), P(o), T, n, n + 8, None, ST], [o]
    run_both(both, "gpu_relu2", relu2, None, exact=True)

    def softcap():
        x = R(T, n) * 40
        return [P(x), T * n, 30.0, ST], [x]
    run_both(both, "gpu_softcap", softcap, None)


def test_moe_bookkeeping(both):
    keep = []
    T, E, U, n = 300, 128, 8, 512

    def router(gate, stride):
        def mk():
            lg, x, w = R(T, E) * 2, R(T, n), R(n) * 0.05
            ids = torch.full((T, stride or U), -5, dtype=torch.int32, device="cuda")
            wts, sg = Z(T, U), Z(T)
            keep.extend([lg, x, w])
            return [P(lg), P(x) if gate else None, P(w) if gate else None, P(ids), P(wts), P(sg) if gate else None, E, U, n, T,
                    ST, stride], [ids, wts, sg.view(T, 1)]
        return mk
    run_both(both, "gpu_moe_router", router(True, 0), None)
    run_both(both, "gpu_moe_router", router(False, U + 1), None)

    def router_sig():
        lg, b = R(T, E) * 2, R(E) * 0.2
        ids, wts = torch.zeros(T, U, dtype=torch.int32, device="cuda"), Z(T, U)
        keep.extend([lg, b])
        return [P(lg), P(b), P(ids), P(wts), E, U, 1, 2.5, T, ST], [ids, wts]
    run_both(both, "gpu_moe_router_sigmoid", router_sig, None)

    def group():
        ids = torch.randint(0, E, (T, U), device="cuda", dtype=torch.int32)
        m = T * U
        mt = min(m, E + m // 32)
        z = lambda k: torch.full((k,), -7, dtype=torch.int32, device="cuda")
        tok, pair, ntl, te, ts, tn = z(m), z(m), z(1), z(mt), z(mt), z(mt)
        keep.append(ids)
        return [P(ids), T, U, E, 32, P(tok), P(pair), P(ntl), P(te), P(ts), P(tn), ST], [tok, pair, ntl, te, ts, tn]
    run_both(both, "gpu_moe_group", group, None, exact=True)

    def combine(scaled, shared):
        def mk():
            down, wts = R(T, U, n), torch.rand(T, U, device="cuda")
            ids = torch.randint(0, E, (T, U), device="cuda", dtype=torch.int32)
            es, sh, sg, out = torch.rand(E, device="cuda") + 0.5, R(T, n), torch.rand(T, device="cuda"), Z(T, n)
            keep.extend([down, wts, ids, es, sh, sg])
            if scaled:
                return [P(down), P(wts), P(sh) if shared else None, P(sg) if shared else None, P(ids), P(es), P(out), U, n, T,
                        ST], [out]
            return [P(down), P(wts), P(sh) if shared else None, P(sg) if shared else None, P(out), U, n, T, ST], [out]
        return mk
    run_both(both, "gpu_moe_combine", combine(False, True), None, exact=True)
    run_both(both, "gpu_moe_combine_scaled", combine(True, False), None, exact=True)

    def ffn_post():
        x, mlp, down, wts = R(T, n), R(T, n), R(T, U, n), torch.rand(T, U, device="cuda")
        ids = torch.randint(0, E, (T, U), device="cuda", dtype=torch.int32)
        es, sc = torch.rand(E, device="cuda") + 0.5, torch.tensor([0.8], device="cuda")
        w = [1 + 0.1 * R(n) for _ in range(4)]
        xo, y = Z(T, n), Z(T, n)
        keep.extend([x, mlp, down, wts, ids, es, sc] + w)
        return [P(x), P(mlp), P(down), P(wts), P(ids), P(es), U, P(w[0]), P(w[1]), P(w[2]), P(sc), P(xo), P(w[3]), P(y), None, n,
                T, 1e-6, ST], [xo, y]
    run_both(both, "gpu_gemma_ffn_post", ffn_post, None)


def test_stream_and_window_ops(both):
    keep = []
    T, hc, n = 7, 4, 768

    def hc_norm():
        res, cur, inj, w = R(T, hc, n), R(T, n), R(T, hc), 1 + 0.1 * R(hc, n)
        ro, y = Z(T, hc, n), Z(T, hc, n)
        keep.extend([res, cur, inj, w])
        return [P(res), P(ro), P(cur), P(inj), P(w), P(y), n, hc, T, 1e-6, None, ST], [ro.view(T * hc, n), y.view(T * hc, n)]
    run_both(both, "gpu_hc_norm", hc_norm, None)

    def hc_lowrank():
        lo, o = R(T, 100) * 3, Z(T, 128)
        keep.append(lo)
        return [P(lo), P(o), 100, 128, T, hc, None, ST], [o]
    run_both(both, "gpu_hc_lowrank", hc_lowrank, None)

    def hc_mix():
        xn, g, o = R(T, hc, n), R(T, hc, n), Z(T, n)
        keep.extend([xn, g])
        return [P(xn), P(g), P(o), n, hc, T, None, ST], [o]
    run_both(both, "gpu_hc_mix", hc_mix, None)

    def ple_gate():
        key, val, res = R(T, hc, n), R(T, n), R(T, hc, n)
        w = [1 + 0.1 * R(hc, n) for _ in range(3)]
        gated, normed = Z(T, hc, n), Z(T, hc, n)
        keep.extend([key, val, res] + w)
        return [P(key), P(val), P(res), P(w[0]), P(w[1]), P(w[2]), P(gated), P(normed), n, hc, T, 1e-6, ST], \
            [gated.view(T * hc, n), normed.view(T * hc, n)]
    run_both(both, "gpu_ple_gate", ple_gate, None)

    def ple_conv():
        m, K, dil = 512, 4, 2
        normed, gated, res, state = R(T, m), R(T, m), R(T, m), R((K - 1) * dil, m)
        w = (R(m, K) * 0.5).half()
        keep.extend([normed, gated, w])
        return [P(normed), P(gated), P(res), P(state), P(w), m, T, K, dil, None, ST], [res, state]
    run_both(both, "gpu_ple_conv", ple_conv, None)

    def mtp_concat():
        e, h, o = R(T, n), R(T, hc, n), Z(T, hc, 2 * n)
        keep.extend([e, h])
        return [P(e), P(h), P(o), n, hc, T, ST], [o.view(T * hc, 2 * n)]
    run_both(both, "gpu_mtp_concat", mtp_concat, None, exact=True)

    n_head, n_group, Tm = 8, 2, 11
    d_inner = n_head * 64
    conv_dim = d_inner + 2 * n_group * 128
    ld = d_inner + conv_dim + n_head

    def mamba_conv():
        zx, st = R(Tm, ld), R(conv_dim, 3)
        w, b, o = R(conv_dim, 4) * 0.5, R(conv_dim) * 0.1, Z(Tm, conv_dim)
        keep.extend([zx, w, b])
        return [P(zx), ld, d_inner, P(st), P(w), P(b), P(o), conv_dim, 4, Tm, ST], [o, st]
    run_both(both, "gpu_mamba_conv", mamba_conv, None)

    def mamba_scan():
        state, xbc, zx = R(n_head, 64, 128) * 0.1, R(Tm, conv_dim), R(Tm, ld)
        dtb, A, D = R(n_head) * 0.5, -torch.rand(n_head, device="cuda") - 0.2, 1 + 0.1 * R(n_head)
        y = Z(Tm, d_inner)
        keep.extend([xbc, zx, dtb, A, D])
        return [P(state), P(xbc), P(zx), ld, d_inner + conv_dim, P(dtb), P(A), P(D), P(y), n_head, d_inner, n_group, Tm, ST], \
            [y, state.view(n_head * 64, 128)]
    run_both(both, "gpu_mamba_scan", mamba_scan, None, exact=True)

    def mamba_gnorm():
        y, zx, w, o = R(Tm, d_inner), R(Tm, ld), 1 + 0.1 * R(d_inner), Z(Tm, d_inner)
        keep.extend([y, zx, w])
        return [P(y), P(zx), ld, P(w), P(o), d_inner, n_group, Tm, 1e-5, None, ST], [o]
    run_both(both, "gpu_mamba_gnorm", mamba_gnorm, None)
