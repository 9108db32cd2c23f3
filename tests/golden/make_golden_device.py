"""Generates tests/golden/device_ops.npz: inputs and outputs of the REFERENCE'S OWN device kernels and launchers for
the layer-op path and its neighbours, run on the CPU.

The reference states these ops only as GPU code (src/gpu_ops.hip with the activation quantiser of src/q8_device.h,
launched by src/gpu_ops.cpp). oracle/Makefile (target ref_emul) compiles exactly those files, unchanged and where they
lie, against the host SIMT emulation headers of oracle/simt/ (threads of a block as host threads, shuffles and barriers
as exchanges between them) into oracle/_ref/libref_emul.so. Run where the reference's source tree is present:

    make -C oracle ref_emul && python tests/golden/make_golden_device.py

The fixtures pin the restatements in oracle/oracle.py (and oracle_ops.c's quantiser) where the reference is absent.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from rocm_hip_b200 import _lib, synth  # noqa: E402  (signatures of the launchers; seeded inputs)

OUT = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(ROOT, "oracle", "_ref", "libref_emul.so")
NAMES = ["gpu_add_rmsnorm", "gpu_swiglu", "gpu_relu2", "gpu_add_normed", "gpu_gemma_attn_post", "gpu_gemma_ffn_post",
         "gpu_geglu", "gpu_softcap", "gpu_moe_combine", "gpu_moe_combine_scaled", "gpu_hc_norm", "gpu_hc_lowrank", "gpu_hc_mix",
         "gpu_ple_gate", "gpu_mtp_concat", "gpu_mamba_gnorm", "gpu_mamba_conv", "gpu_mamba_scan", "gpu_ple_conv",
         "gpu_moe_router", "gpu_moe_router_sigmoid", "gpu_moe_group"]


def load():
    lib = C.CDLL(LIB)
    lib.gpu_ops_init.restype, lib.gpu_ops_init.argtypes = C.c_int, [C.c_char_p]
    for n in NAMES:
        getattr(lib, n).restype, getattr(lib, n).argtypes = _lib.SIGNATURES[n]
    assert lib.gpu_ops_init(b"gpu_ops.co") == 0
    return lib


def P(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def q8_bufs(K, xh_bf16=1):
    b = dict(q0=np.zeros(K, np.int8), d0=np.zeros(K // 32 + 1, np.float32), qK=np.zeros(K, np.int8),
             dK=np.zeros(K // 256 + 1, np.float32), bsK=np.zeros(K // 16 + 1, np.int32), s0=np.zeros(K // 32 + 1, np.int32),
             xh=np.zeros(K, np.uint16))
    g = lambda k: b[k].ctypes.data
    return _lib.qmatvec_q8(g("q0"), g("d0"), g("qK"), g("dK"), g("bsK"), g("s0"), K, g("xh"), xh_bf16), b


def main():
    lib = load()
    f = lambda name, *shape, mean=0.0, std=1.0: synth.normal(7, "dev." + name, 0, int(np.prod(shape)), mean, std).reshape(shape)
    out = {}

    # ---- add_rmsnorm_rows (T > 1, n % 256 == 0) and the split kernel (T == 1; odd width), with and without add / q8
    for tag, T, n, add, q8 in (("rows", 3, 512, True, True), ("rows_noadd", 2, 1024, False, True),
                               ("split", 1, 768, True, True), ("odd", 2, 1000, True, False)):
        x, a, w = f(tag + ".x", T, n), f(tag + ".a", T, n), f(tag + ".w", n, mean=1.0, std=0.1)
        xo, y = np.zeros_like(x), np.zeros_like(x)
        s, b = q8_bufs(T * n) if q8 else (None, {})
        assert lib.gpu_add_rmsnorm(P(x), P(a) if add else None, P(xo), P(w), P(y), n, T, 1e-6, C.byref(s) if q8 else None, None) == 0
        out.update({f"norm_{tag}_x": x, f"norm_{tag}_w": w, f"norm_{tag}_y": y})
        if add:
            out.update({f"norm_{tag}_a": a, f"norm_{tag}_xo": xo})
        for k, v in b.items():
            out[f"norm_{tag}_{k}"] = v

    # ---- swiglu with side outputs: whole Q8_K blocks and a last partial one (n % 32 == 0)
    for tag, n in (("full", 1024), ("tail", 2 * 256 + 96)):
        g, u = f("sw.g" + tag, n, std=2.0), f("sw.u" + tag, n)
        o = np.zeros_like(g)
        s, b = q8_bufs((n + 255) // 256 * 256, xh_bf16=0)
        assert lib.gpu_swiglu(P(g), P(u), P(o), n, C.byref(s), None) == 0
        out.update({f"swiglu_{tag}_g": g, f"swiglu_{tag}_u": u, f"swiglu_{tag}_out": o})
        for k, v in b.items():
            out[f"swiglu_{tag}_{k}"] = v

    # ---- relu2 on values whose squares are exact in fp32: its output is known to the bit, so the side outputs pin
    #      the quantisation rules alone (ties, a zero block, equal magnitudes of both signs, a block maximum of -x)
    rows, h = 2, 512
    v = np.round(f("relu.x", rows, h) * 64).astype(np.float32) / np.float32(8)
    v[0, 32:64] = 0
    v[0, 64], v[0, 65] = 9.0, 9.0
    v[1, :256] = -np.abs(v[1, :256])
    v[1, 300:320] = 7.5
    o = np.zeros((rows, h), np.float32)
    s, b = q8_bufs(rows * h)
    assert lib.gpu_relu2(P(v), P(o), rows, h, h, C.byref(s), None) == 0
    out.update(relu2_x=v, relu2_out=o)
    for k, vv in b.items():
        out["relu2_" + k] = vv

    # ---- the Gemma-4 chains and their neighbours
    T, n, U, E = 3, 512, 4, 16
    base, a, w, sc = f("an.base", T, n), f("an.a", T, n), f("an.w", n, mean=1.0, std=0.1), np.array([0.7], np.float32)
    o = np.zeros_like(base)
    assert lib.gpu_add_normed(P(base), P(a), P(w), P(sc), P(o), n, T, 1e-6, None) == 0
    out.update(add_normed_base=base, add_normed_a=a, add_normed_w=w, add_normed_scale=sc, add_normed_out=o)

    x, a, wa, w1, w2 = f("ap.x", T, n), f("ap.a", T, n), f("ap.wa", n, mean=1.0, std=0.1), f("ap.w1", n, mean=1.0, std=0.1), f("ap.w2", n, mean=1.0, std=0.1)
    xo, y1, y2 = np.zeros_like(x), np.zeros_like(x), np.zeros_like(x)
    assert lib.gpu_gemma_attn_post(P(x), P(a), P(wa), P(xo), P(w1), P(y1), None, P(w2), P(y2), n, T, 1e-6, None) == 0
    out.update(attn_post_x=x, attn_post_a=a, attn_post_wa=wa, attn_post_w1=w1, attn_post_w2=w2, attn_post_xo=xo,
               attn_post_y1=y1, attn_post_y2=y2)

    x, mlp, down = f("fp.x", T, n), f("fp.mlp", T, n), f("fp.down", T, U, n)
    wts = np.abs(f("fp.wts", T, U)).astype(np.float32)
    ids = synth.randint(7, "dev.fp.ids", 0, T * U, 0, E).astype(np.int32).reshape(T, U)
    es = (1 + 0.1 * f("fp.es", E)).astype(np.float32)
    w1, w2, wp, wn = (f("fp.w%d" % i, n, mean=1.0, std=0.1) for i in range(4))
    xo, y = np.zeros_like(x), np.zeros_like(x)
    assert lib.gpu_gemma_ffn_post(P(x), P(mlp), P(down), P(wts), P(ids), P(es), U, P(w1), P(w2), P(wp), P(sc), P(xo), P(wn),
                                  P(y), None, n, T, 1e-6, None) == 0
    out.update(ffn_post_x=x, ffn_post_mlp=mlp, ffn_post_down=down, ffn_post_wts=wts, ffn_post_ids=ids, ffn_post_es=es,
               ffn_post_w1=w1, ffn_post_w2=w2, ffn_post_wp=wp, ffn_post_wn=wn, ffn_post_scale=sc, ffn_post_xo=xo, ffn_post_y=y)

    comb = np.zeros((T, n), np.float32)
    shared, sg = f("mc.shared", T, n), np.abs(f("mc.sg", T)).astype(np.float32)
    assert lib.gpu_moe_combine_scaled(P(down), P(wts), P(shared), P(sg), P(ids), P(es), P(comb), U, n, T, None) == 0
    out.update(combine_shared=shared, combine_sg=sg, combine_out=comb)

    gu = f("gg.gu", T, 2 * n, std=2.0)
    o = np.zeros((T, n), np.float32)
    assert lib.gpu_geglu(P(gu), C.c_void_p(gu.ctypes.data + 4 * n), P(o), T, n, 2 * n, 2 * n, None, None) == 0
    out.update(geglu_gu=gu, geglu_out=o)

    xs = (f("sc.x", T * n) * 40).astype(np.float32)
    capped = xs.copy()
    assert lib.gpu_softcap(P(capped), T * n, 30.0, None) == 0
    out.update(softcap_x=xs, softcap_out=capped)

    neighbours(lib, out, f)
    attn_prep(lib, out, f)
    phase3(lib, out)
    np.savez_compressed(os.path.join(OUT, "device_ops.npz"), **out)
    print("wrote device_ops.npz:", len(out), "arrays,", os.path.getsize(os.path.join(OUT, "device_ops.npz")) // 1024, "KB")


def neighbours(lib, out, f):
    """The other row-parallel launchers of the module: hyper-connection ops, PLE gate / conv, Mamba-2 ops, the routers."""
    T, hc, n = 3, 2, 256
    res, cur, inj, w = f("hc.res", T, hc, n), f("hc.cur", T, n), f("hc.inj", T, hc) * 3, f("hc.w", hc, n, mean=1.0, std=0.1)
    ro, y = np.zeros_like(res), np.zeros_like(res)
    s, b = q8_bufs(T * hc * n)
    assert lib.gpu_hc_norm(P(res), P(ro), P(cur), P(inj), P(w), P(y), n, hc, T, 1e-6, C.byref(s), None) == 0
    out.update(hc_res=res, hc_cur=cur, hc_inj=inj, hc_w=w, hc_res_out=ro, hc_y=y, hc_q0=b["q0"], hc_d0=b["d0"],
               hc_qK=b["qK"], hc_dK=b["dK"], hc_bsK=b["bsK"], hc_s0=b["s0"], hc_xh=b["xh"])

    lo, np_ = f("lr.lo", T, 100) * 4, 128
    o = np.full((T, np_), -1.0, np.float32)
    assert lib.gpu_hc_lowrank(P(lo), P(o), 100, np_, T, 4, None, None) == 0
    out.update(lowrank_lo=lo, lowrank_out=o)

    xn, gate = f("mx.xn", T, hc, n), f("mx.gate", T, hc, n) * 2
    o = np.zeros((T, n), np.float32)
    assert lib.gpu_hc_mix(P(xn), P(gate), P(o), n, hc, T, None, None) == 0
    out.update(mix_xn=xn, mix_gate=gate, mix_out=o)

    key, rs, val = f("pg.key", T, hc, n), f("pg.res", T, hc, n), f("pg.val", T, n)
    rs[0, 0], rs[1, 0] = -key[0, 0], key[1, 0]
    wk, wq, wc = (f("pg.w%d" % i, hc, n, mean=1.0, std=0.1) for i in range(3))
    gated, normed = np.zeros_like(key), np.zeros_like(key)
    assert lib.gpu_ple_gate(P(key), P(val), P(rs), P(wk), P(wq), P(wc), P(gated), P(normed), n, hc, T, 1e-6, None) == 0
    out.update(ple_key=key, ple_res=rs, ple_val=val, ple_wk=wk, ple_wq=wq, ple_wc=wc, ple_gated=gated, ple_normed=normed)

    e, h = f("mt.e", T, n), f("mt.h", T, hc, n)
    o = np.zeros((T, hc, 2 * n), np.float32)
    assert lib.gpu_mtp_concat(P(e), P(h), P(o), n, hc, T, None) == 0
    out.update(mtp_e=e, mtp_h=h, mtp_out=o)

    d_inner, n_group = 512, 2
    ld = d_inner + 2 * 128 + 64
    yv, zx, w = f("gn.y", T, d_inner), f("gn.zx", T, ld) * 2, f("gn.w", d_inner, mean=1.0, std=0.1)
    o = np.zeros((T, d_inner), np.float32)
    assert lib.gpu_mamba_gnorm(P(yv), P(zx), ld, P(w), P(o), d_inner, n_group, T, 1e-5, None, None) == 0
    out.update(gnorm_y=yv, gnorm_zx=zx, gnorm_w=w, gnorm_out=o)

    conv_dim, d_conv, x_off, Tc = 320, 4, 64, 5
    ld = x_off + conv_dim + 16
    zx, st = f("mv.zx", Tc, ld), f("mv.st", conv_dim, d_conv - 1)
    w, bias = f("mv.w", conv_dim, d_conv, std=0.5), f("mv.b", conv_dim, std=0.1)
    st_io, o = st.copy(), np.zeros((Tc, conv_dim), np.float32)
    assert lib.gpu_mamba_conv(P(zx), ld, x_off, P(st_io), P(w), P(bias), P(o), conv_dim, d_conv, Tc, None) == 0
    out.update(conv_zx=zx, conv_state=st, conv_w=w, conv_bias=bias, conv_out=o, conv_state_out=st_io)

    n_head, n_group, Ts = 4, 2, 3
    d_inner = n_head * 64
    conv_dim = d_inner + 2 * n_group * 128
    dt_off = d_inner + conv_dim
    ld = dt_off + n_head
    xbc, zx = f("ms.xbc", Ts, conv_dim), f("ms.zx", Ts, ld)
    zx[0, dt_off] = 25.0
    state = f("ms.state", n_head, 64, 128) * np.float32(0.1)
    dt_b, D = f("ms.dtb", n_head, std=0.5), f("ms.D", n_head, mean=1.0, std=0.1)
    A = -np.abs(f("ms.A", n_head, mean=1.0, std=0.3)).astype(np.float32)
    st_io, o = state.copy(), np.zeros((Ts, d_inner), np.float32)
    assert lib.gpu_mamba_scan(P(st_io), P(xbc), P(zx), ld, dt_off, P(dt_b), P(A), P(D), P(o), n_head, d_inner, n_group, Ts, None) == 0
    out.update(scan_xbc=xbc, scan_zx=zx, scan_state=state, scan_dtb=dt_b, scan_A=A, scan_D=D, scan_y=o, scan_state_out=st_io)

    from oracle import oracle
    m, K, dil, Tp = 128, 4, 2, 6
    H = (K - 1) * dil
    nm, gt, rs, st = f("pc.n", Tp, m), f("pc.g", Tp, m), f("pc.r", Tp, m), f("pc.s", H, m)
    wb = oracle.f32_to_f16(f("pc.w", m, K, std=0.5)).reshape(m, K)
    rs_io, st_io = rs.copy(), st.copy()
    mids = [np.full((H, m), -9.0, np.float32) for _ in range(3)]
    arr = (C.c_void_p * 3)(*[a.ctypes.data for a in mids])
    assert lib.gpu_ple_conv(P(nm), P(gt), P(rs_io), P(st_io), P(wb), m, Tp, K, dil, C.cast(arr, C.c_void_p), None) == 0
    out.update(pconv_normed=nm, pconv_gated=gt, pconv_res=rs, pconv_state=st, pconv_w=wb, pconv_res_out=rs_io,
               pconv_state_out=st_io, pconv_mid=np.stack(mids))

    Tr, ne, nu, nx = 9, 64, 6, 256
    lg = (f("rt.l", Tr, ne) * 2).astype(np.float32)
    lg[0, 5] = lg[0, 9]                                       # equal logits: the lower index wins
    x, w = f("rt.x", Tr, nx), f("rt.w", nx, std=0.05)
    ids, wts, sg = np.zeros((Tr, nu), np.int32), np.zeros((Tr, nu), np.float32), np.zeros(Tr, np.float32)
    assert lib.gpu_moe_router(P(lg), P(x), P(w), P(ids), P(wts), P(sg), ne, nu, nx, Tr, None, 0) == 0
    out.update(router_logits=lg, router_x=x, router_w=w, router_ids=ids, router_wts=wts, router_sg=sg)
    bias = f("rt.b", ne, std=0.2)
    ids2, wts2 = np.zeros((Tr, nu), np.int32), np.zeros((Tr, nu), np.float32)
    assert lib.gpu_moe_router_sigmoid(P(lg), P(bias), P(ids2), P(wts2), ne, nu, 1, 2.5, Tr, None) == 0
    out.update(sigrouter_bias=bias, sigrouter_ids=ids2, sigrouter_wts=wts2)

    tile, npair = 4, Tr * nu
    mt = min(npair, ne + npair // tile)
    tok, pair = np.full(npair, -7, np.int32), np.full(npair, -7, np.int32)
    ntl, te, ts, tn = np.zeros(1, np.int32), np.full(mt, -7, np.int32), np.full(mt, -7, np.int32), np.full(mt, -7, np.int32)
    assert lib.gpu_moe_group(P(ids), Tr, nu, ne, tile, P(tok), P(pair), P(ntl), P(te), P(ts), P(tn), None) == 0
    out.update(group_tile=np.array([tile], np.int32), group_tok=tok, group_pair=pair, group_n_tiles=ntl, group_tile_e=te,
               group_tile_start=ts, group_tile_n=tn)


def launch(lib, name, grid, block, args):
    """One launch of a kernel of the emulated module by name, arguments as ctypes values in the kernel's order."""
    fn = C.c_void_p()
    lib.hipModuleGetFunction.argtypes = [C.POINTER(C.c_void_p), C.c_void_p, C.c_char_p]
    lib.hipModuleLaunchKernel.argtypes = [C.c_void_p] + [C.c_uint] * 7 + [C.c_void_p] * 3
    assert lib.hipModuleGetFunction(C.byref(fn), None, name.encode()) == 0, name
    ptrs = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
    assert lib.hipModuleLaunchKernel(fn, grid[0], grid[1], 1, block, 1, 1, 0, None, ptrs, None) == 0


def attn_prep(lib, out, f):
    """attn_prep_<D> (src/attention.hip:266-300, launched as src/attention.cpp:150-156 does: grid (n_q + n_kv, T), block
    D): q / k norm + RoPE, the Hadamard rotation, FP16 / Q8_0 / Q4_0 cache rows. 'exact' cases switch the norm and the
    RoPE off, so every stored byte follows from the inputs by exactly rounded steps; 'chain' cases run everything."""
    vp, ci, cf, cll = C.c_void_p, C.c_int, C.c_float, C.c_longlong
    for tag, D, nq, nkv, T, chain, gated, kvq, pos0 in (
            ("exact_q8", 128, 4, 2, 3, 0, 0, 1, 7), ("exact_q4", 128, 4, 2, 3, 0, 0, 2, 7), ("exact_q8_rot", 128, 4, 2, 3, 0, 0, 1 | 4, 7),
            ("exact_q4_rot", 256, 2, 1, 2, 0, 0, 2 | 4, 7), ("exact_q8_rot512", 512, 2, 1, 2, 0, 0, 1 | 4, 7),
            ("chain_f16", 128, 4, 2, 5, 1, 0, 0, 7), ("chain_gated_f16", 256, 2, 1, 3, 1, 1, 0, 7),
            ("chain_q8_rot", 128, 4, 2, 4, 1, 0, 1 | 4, 7), ("chain_q4_rot", 64, 2, 2, 3, 1, 0, 2 | 4, 7),
            # the position the reference's own test compares its kernel with its CPU ops at (tests/forward_verify.cpp:835-853)
            ("chain_pos2499", 128, 4, 2, 2, 1, 0, 0, 2499)):
        qs = 2 * D if gated else D
        q, k, v = f(tag + ".q", T, nq * qs) * 2, f(tag + ".k", T, nkv * D) * 3, f(tag + ".v", T, nkv * D) * 3
        if not chain:
            k[0, :32] = 0.0
            k[1, 32:64] = np.linspace(-2, 2, 32, dtype=np.float32)
            v[0, 5] = 1e30
            v[1, 64:96] = -np.abs(v[1, 64:96])
        qn, kn = f(tag + ".qn", D, mean=1.0, std=0.1), f(tag + ".kn", D, mean=1.0, std=0.1)
        n_vals, kq = nkv * D, kvq & 3
        kv_stride = n_vals if kq == 0 else n_vals * (17 if kq == 1 else 9) // 32      # in 2-byte units
        n_ctx = pos0 + T + 2
        K, V = np.full(n_ctx * kv_stride, 0x5A5A, np.uint16), np.full(n_ctx * kv_stride, 0x5A5A, np.uint16)
        q_out = np.zeros((T, nq * D), np.float32)
        n_rot = D if chain else 0
        args = [vp(q.ctypes.data), vp(k.ctypes.data), vp(v.ctypes.data), vp(qn.ctypes.data), vp(kn.ctypes.data),
                vp(q_out.ctypes.data), vp(K.ctypes.data), vp(V.ctypes.data), ci(kv_stride), ci(30), cll(0), ci(nq), ci(nkv),
                ci(n_rot), ci(pos0), cf(1e6), cf(1e-6), ci(gated), ci(n_rot // 2), ci(0), ci(chain), ci(kvq), vp(None), vp(None),
                vp(None), ci(0), vp(None)]
        launch(lib, "attn_prep_%d" % D, (nq + nkv, T), D, args)
        out.update({f"prep_{tag}_q": q, f"prep_{tag}_k": k, f"prep_{tag}_v": v, f"prep_{tag}_qn": qn, f"prep_{tag}_kn": kn,
                    f"prep_{tag}_q_out": q_out, f"prep_{tag}_K": K, f"prep_{tag}_V": V,
                    f"prep_{tag}_cfg": np.array([D, nq, nkv, T, chain, gated, kvq, pos0, kv_stride], np.int32)})


def phase3(lib, out):
    """The FP16 component kernels on the inputs of the reference's own test programs: "rmsnorm" (src/layernorm.hip) on
    the sweep of tests/layernorm_verify.cpp:64-66,139 (LCG seed 7 per shape, eps 1e-5, grid = tokens, block = 32) and
    "rope_rotate_half" (src/rope_embedding.hip) on the sweep of tests/rope_verify.cpp:69-81,152-164 (seed 13, positions
    from the second LCG, theta 1e4, tables built in double and stored fp32)."""
    from oracle import oracle
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    for tokens, embd in ((8, 17), (32, 64), (5, 4096), (1, 96), (7, 48)):
        rng = oracle.Lcg(7)
        x = np.array([rng.rnd(-3.0, 3.0) for _ in range(tokens * embd)], dtype=np.float32)
        gam = np.array([rng.rnd(0.5, 1.5) for _ in range(embd)], dtype=np.float32)
        xh, gh = oracle.f32_to_f16(x).reshape(tokens, embd), oracle.f32_to_f16(gam)
        y, y1 = np.zeros_like(xh), np.zeros_like(xh)
        launch(lib, "rmsnorm", (tokens, 1), 32, [vp(xh.ctypes.data), vp(gh.ctypes.data), vp(y.ctypes.data), ci(tokens), ci(embd), cf(1e-5)])
        launch(lib, "rmsnorm", (tokens, 1), 32, [vp(xh.ctypes.data), vp(None), vp(y1.ctypes.data), ci(tokens), ci(embd), cf(1e-5)])
        out.update({f"p3norm_{tokens}x{embd}_x": xh, f"p3norm_{tokens}x{embd}_gamma": gh, f"p3norm_{tokens}x{embd}_y": y,
                    f"p3norm_{tokens}x{embd}_y_nogamma": y1})
    state, pos = 99, []
    for _ in range(64):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        pos.append(1 + (state >> 8) % 4096)
    pos = np.array(pos, dtype=np.int32)
    for rows, dim in ((16, 16), (5, 32), (64, 128)):
        rng = oracle.Lcg(13)
        x = oracle.f32_to_f16(np.array([rng.rnd(-3.0, 3.0) for _ in range(rows * dim)], dtype=np.float32)).reshape(rows, dim)
        c, s = oracle.rope_tables(pos[:rows], dim, 10000.0)
        y = np.zeros_like(x)
        launch(lib, "rope_rotate_half", (rows, 1), 32, [vp(x.ctypes.data), vp(c.ctypes.data), vp(s.ctypes.data), vp(y.ctypes.data),
                                                        ci(rows), ci(dim // 2)])
        out.update({f"p3rope_{rows}x{dim}_x": x, f"p3rope_{rows}x{dim}_c": c, f"p3rope_{rows}x{dim}_s": s, f"p3rope_{rows}x{dim}_y": y})


if __name__ == "__main__":
    main()
