"""numpy front end of the CPU checkers. TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the
benchmark's CPU baseline, never by the product package.

``port``  = oracle/liboracle.so, the restatement of the reference's arithmetic (oracle_ops.c).
``ref``   = oracle/_ref/libref_cpu.so, the reference's own qwen_ops.cpp / quant_types.cpp compiled from its source
            tree (present when that tree was available at build time; the built file travels with the repository).
Both export the row-parallel cpu_* runner of cpu_rows.cpp.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(HERE, "liboracle.so")
REF_PATH = os.path.join(HERE, "_ref", "libref_cpu.so")

Q4_0, Q8_0 = 2, 8
F32, F16, Q4_1, Q5_0, Q5_1, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 3, 6, 7, 12, 13, 14, 30
# (values per block, bytes per block) of every row format the embedding gather decodes (src/quant_types.cpp:583-598)
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24),
         Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}

_p, _i, _ll, _f, _sz = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_size_t


def build():
    """Compiles liboracle.so and, when the reference's sources are present, _ref/libref_cpu.so."""
    subprocess.run(["make", "-s", "-C", HERE], check=True, stdout=subprocess.DEVNULL)


_CPU_SIGS = {
    "cpu_hardware_threads": (_i, []),
    "cpu_is_reference": (_i, []),
    "cpu_add_rmsnorm": (None, [_p, _p, _p, _p, _p, _i, _i, _f, _i]),
    "cpu_swiglu": (None, [_p, _p, _p, _ll, _i]),
    "cpu_qk_norm_rope": (None, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _i, _i, _f, _f, _i, _i, _i]),
    "cpu_embed_rows": (_i, [_i, _p, _sz, _i, _p, _p, _i, _i, _f, _i]),
}
_PORT_SIGS = {
    "orc_fp16_to_fp32": (_f, [C.c_uint16]),
    "orc_fp32_to_fp16": (C.c_uint16, [_f]),
    "orc_fp32_to_bf16": (C.c_uint16, [_f]),
    "orc_rmsnorm": (None, [_p, _p, _p, _i, _f]),
    "orc_add_rmsnorm": (None, [_p, _p, _p, _p, _p, _i, _i, _f]),
    "orc_add_rmsnorm_bf16": (None, [_p, _p, _p, _p, _p, _i, _i, _f]),
    "orc_silu": (_f, [_f]),
    "orc_swiglu": (None, [_p, _p, _p, _ll]),
    "orc_swiglu_bf16": (None, [_p, _p, _p, _ll]),
    "orc_swiglu_strided": (None, [_p, _p, _p, _i, _i, _ll, _ll]),
    "orc_rope_neox": (None, [_p, _i, _i, _f]),
    "orc_rope_neox_ex": (None, [_p, _i, _i, _i, _f, _p]),
    "orc_qk_norm_rope": (None, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _i, _f, _f, _i, _p, _i]),
    "orc_qk_norm_rope_bf16": (None, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _i, _f, _f, _i, _p, _i]),
    "orc_row_size": (_sz, [_i, _ll]),
    "orc_to_float": (_i, [_i, _p, _p, _ll]),
    "orc_embed_rows": (_i, [_i, _p, _sz, _i, _p, _p, _i, _i, _f]),
    "orc_embed_rows_bf16": (_i, [_i, _p, _sz, _i, _p, _p, _i, _i, _f]),
    "orc_rmsnorm_f16": (None, [_p, _p, _p, _i, _i, _f]),
    "orc_rope_tables": (None, [_p, _i, _i, _f, _p, _p]),
    "orc_rope_rotate_half_f16": (None, [_p, _p, _p, _p, _i, _i]),
    "orc_lcg": (_f, [C.POINTER(C.c_uint32), _f, _f]),
    "orc_quantize_q8": (None, [_p, _ll, _p, _p, _p, _p, _p, _p, _p, _i]),
}
_REF_SIGS = {
    "ref_qwen_rmsnorm": (None, [_p, _p, _p, _i, _f]),
    "ref_qwen_rope_neox": (None, [_p, _i, _i, _f]),
    "ref_qwen_silu": (_f, [_f]),
    "qt_to_float": (_i, [_i, _p, _p, C.c_int64]),
    "qt_row_size": (_sz, [_i, C.c_int64]),
    "qt_fp16_to_fp32": (_f, [C.c_uint16]),
    "qt_bf16_to_fp32": (_f, [C.c_uint16]),
}


def _bind(lib, sigs):
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


_port = _ref = None


def port():
    global _port
    if _port is None:
        if not os.path.exists(PORT_PATH):
            build()
        _port = _bind(_bind(C.CDLL(PORT_PATH), _PORT_SIGS), _CPU_SIGS)
    return _port


def have_ref():
    return os.path.exists(REF_PATH)


def ref():
    global _ref
    if _ref is None:
        if not have_ref():
            raise FileNotFoundError(REF_PATH)
        _ref = _bind(_bind(C.CDLL(REF_PATH), _REF_SIGS), _CPU_SIGS)
    return _ref


def ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


# ---------------------------------------------------------------- conversions (vectorised numpy equivalents)

def bf16_to_f32(u16):
    return (np.asarray(u16, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x):
    """Round to nearest even on the bit pattern (src/q8_device.h:39-40)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def f16_to_f32(u16):
    return np.asarray(u16, dtype=np.uint16).view(np.float16).astype(np.float32)


def f32_to_f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


# ---------------------------------------------------------------- ops on numpy arrays (restatement)

def add_rmsnorm(x_in, add, w, eps):
    """fp32 [T][n] -> (x_out or None, y)."""
    x_in = _c(x_in, np.float32)
    T, n = x_in.shape
    add = _c(add, np.float32)
    w = _c(w, np.float32)
    y = np.empty_like(x_in)
    x_out = np.empty_like(x_in) if add is not None else None
    port().orc_add_rmsnorm(ptr(x_in), ptr(add), ptr(x_out), ptr(w), ptr(y), n, T, eps)
    return x_out, y


def add_rmsnorm_bf16(x_in, add, w, eps):
    x_in = _c(x_in, np.uint16)
    T, n = x_in.shape
    add = _c(add, np.uint16)
    w = _c(w, np.float32)
    y = np.empty_like(x_in)
    x_out = np.empty_like(x_in) if add is not None else None
    port().orc_add_rmsnorm_bf16(ptr(x_in), ptr(add), ptr(x_out), ptr(w), ptr(y), n, T, eps)
    return x_out, y


def swiglu(g, u):
    g, u = _c(g, np.float32), _c(u, np.float32)
    out = np.empty_like(g)
    port().orc_swiglu(ptr(g), ptr(u), ptr(out), g.size)
    return out


def swiglu_bf16(g, u):
    g, u = _c(g, np.uint16), _c(u, np.uint16)
    out = np.empty_like(g)
    port().orc_swiglu_bf16(ptr(g), ptr(u), ptr(out), g.size)
    return out


def qk_norm_rope(qfull, k, q_norm, k_norm, n_q, n_kv, D, n_rot, rot_pairs, positions, pos0, base, eps, gated=0,
                 ff=None, do_norm=1, bf16=False):
    """qfull [T][n_q * (2D if gated else D)], k [T][n_kv * D] (fp32, or uint16 bf16 bits) -> (q_out, k_out)."""
    dt = np.uint16 if bf16 else np.float32
    qfull, k = _c(qfull, dt), _c(k, dt)
    T = qfull.shape[0] if qfull is not None else k.shape[0]
    q_out = np.empty((T, n_q * D), dtype=dt)
    k_out = np.empty((T, n_kv * D), dtype=dt)
    positions = _c(positions, np.int32)
    q_norm, k_norm, ff = _c(q_norm, np.float32), _c(k_norm, np.float32), _c(ff, np.float32)
    fn = port().orc_qk_norm_rope_bf16 if bf16 else port().orc_qk_norm_rope
    fn(ptr(qfull), ptr(k), ptr(q_norm), ptr(k_norm), ptr(q_out), ptr(k_out), n_q, n_kv, D, n_rot, rot_pairs,
       ptr(positions), pos0, T, base, eps, gated, ptr(ff), do_norm)
    return q_out, k_out


def embed_rows(qtype, table, row_bytes, vocab, tokens, E, scale=1.0, bf16=False):
    """table: uint8 array. Returns (status, out [T][E])."""
    tokens = _c(tokens, np.int32)
    T = tokens.size
    out = np.zeros((T, E), dtype=np.uint16 if bf16 else np.float32)
    fn = port().orc_embed_rows_bf16 if bf16 else port().orc_embed_rows
    st = fn(qtype, ptr(table), row_bytes, vocab, ptr(tokens), ptr(out), E, T, scale)
    return st, out


def rmsnorm_f16(x, gamma, eps):
    x = _c(x, np.uint16)
    T, n = x.shape
    gamma = _c(gamma, np.uint16)
    y = np.empty_like(x)
    port().orc_rmsnorm_f16(ptr(x), ptr(gamma), ptr(y), T, n, eps)
    return y


def rope_tables(positions, dim, theta):
    positions = _c(positions, np.int32)
    R, H = positions.size, dim // 2
    c, s = np.empty((R, H), np.float32), np.empty((R, H), np.float32)
    port().orc_rope_tables(ptr(positions), R, dim, theta, ptr(c), ptr(s))
    return c, s


def rope_rotate_half_f16(x, ctab, stab):
    x = _c(x, np.uint16)
    R, dim = x.shape
    y = np.empty_like(x)
    port().orc_rope_rotate_half_f16(ptr(x), ptr(_c(ctab, np.float32)), ptr(_c(stab, np.float32)), ptr(y), R, dim // 2)
    return y


def quantize_q8(x, xh=None, int8=True):
    """Side outputs of a finished vector x (fp32, size % 256 == 0). Returns a dict of arrays."""
    x = _c(x, np.float32).ravel()
    K = x.size
    o = {}
    if int8:
        o.update(q0=np.zeros(K, np.int8), d0=np.zeros(K // 32, np.float32), s0=np.zeros(K // 32, np.int32),
                 qK=np.zeros(K, np.int8), dK=np.zeros(K // 256, np.float32), bsK=np.zeros(K // 16, np.int32))
    if xh:
        o["xh"] = np.zeros(K, np.uint16)
    port().orc_quantize_q8(ptr(x), K, ptr(o.get("q0")), ptr(o.get("d0")), ptr(o.get("s0")), ptr(o.get("qK")),
                           ptr(o.get("dK")), ptr(o.get("bsK")), ptr(o.get("xh")), 1 if xh == "bf16" else 0)
    return o


def hadamard_k(D):
    """Block of the q / K rotation: 64, doubled while it divides D (src/attention.hip:243-247)."""
    r = 64
    while D % (2 * r) == 0:
        r *= 2
    return r


def hadamard_rot(x, N):
    """The reference's hadamard_rot (src/attention.hip:251-263) on the last axis in blocks of N: butterflies
    s = 1, 2, ..., N / 2 in that order, value d becoming (d & s) ? v[d ^ s] - v[d] : v[d] + v[d ^ s] in fp32, then a
    multiply by the float 1 / sqrtf(N)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    v = x.reshape(-1, N).copy()
    d = np.arange(N)
    s = 1
    while s < N:
        y = v[:, d ^ s]
        v = np.where((d & s) != 0, y - v, v + y).astype(np.float32)
        s <<= 1
    r = np.float32(1.0) / np.sqrt(np.float32(N))
    return (v * r).astype(np.float32).reshape(x.shape)


def kv_quant_rows(x, kq):
    """Quantised KV cache rows of x [T][n_vals] fp32 (n_vals % 32 == 0), by the reference's kvq_store
    (src/attention.hip:159-178; row layout :44-50), every float32 operation rounded on its own. Returns (values,
    scales): kq 1 (Q8_0) int8 [T][n_vals], kq 2 (Q4_0) uint8 [T][n_vals / 2] with byte 4 j + k holding values 8 j + k
    (low nibble) and 8 j + k + 4 (high); scales are fp16 bit patterns [T][n_vals / 32]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, n = x.shape
    b = x.reshape(T, n // 32, 32)
    one = np.float32(1.0)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        amax = np.abs(b).max(axis=2, keepdims=True)
        if kq == 1:
            d = amax / np.float32(127.0)
            q = np.where(d != 0, b * (one / d), np.float32(0.0)).astype(np.float32)
            vals = np.rint(q).astype(np.int32).astype(np.int8).reshape(T, n)
        else:
            m = np.where(np.abs(b) == amax, b, -np.inf).astype(np.float32).max(axis=2, keepdims=True)
            d = (m / np.float32(-8.0)).astype(np.float32)
            v = np.where(d != 0, (b * (one / d)).astype(np.float32) + np.float32(8.5), np.float32(8.0)).astype(np.float32)
            nib = np.minimum(15, v.astype(np.int32)).astype(np.uint8).reshape(T, n // 8, 8)   # (int) truncates
            vals = (nib[:, :, :4] | (nib[:, :, 4:] << 4)).astype(np.uint8).reshape(T, n // 2)
        scales = f32_to_f16(d.reshape(T, n // 32)).reshape(T, n // 32)   # a huge scale overflows to inf, as __float2half
    return vals, scales


def _row_inv_rms(v, eps):
    """(float)(1 / sqrt(sum v^2 / n + eps)) per row with the sum in double, the CPU reference's accumulation
    (src/qwen_ops.cpp:8-11) that this build's kernels keep for every RMSNorm."""
    v = np.asarray(v, dtype=np.float32)
    ss = (v.astype(np.float64) ** 2).sum(axis=1, keepdims=True)
    return (1.0 / np.sqrt(ss / v.shape[1] + np.float64(np.float32(eps)))).astype(np.float32)


def add_normed(base, a, w, scale, eps):
    """out = (base + RMSNorm(a) * w) * scale, fp32 operations one by one in the order of the reference's add_normed
    kernel (src/gpu_ops.hip:521-549): ((a * inv) * w + base) * s."""
    base, a, w = (np.asarray(t, dtype=np.float32) for t in (base, a, w))
    s = np.float32(1.0 if scale is None else scale)
    return ((base + (a * _row_inv_rms(a, eps)) * w) * s).astype(np.float32)


def gemma_attn_post(x, a, w_a, w1, w2, eps):
    """x_out = x + RMSNorm(a) * w_a; y1 = RMSNorm(x_out) * w1; y2 = RMSNorm(x_out) * w2 or None
    (src/gpu_ops.hip:577-606), fp32 operations one by one."""
    x, a, w_a, w1 = (np.asarray(t, dtype=np.float32) for t in (x, a, w_a, w1))
    x_out = (x + (a * _row_inv_rms(a, eps)) * w_a).astype(np.float32)
    vn = (x_out * _row_inv_rms(x_out, eps)).astype(np.float32)
    return x_out, (vn * w1).astype(np.float32), None if w2 is None else (vn * np.asarray(w2, np.float32)).astype(np.float32)


def _top_rounds(keys, weights, n_used):
    """n_used rounds of 'largest remaining key, lowest index among equals' (src/gpu_ops.hip:150-182)."""
    keys = np.array(keys, dtype=np.float32)
    T = keys.shape[0]
    ids = np.empty((T, n_used), dtype=np.int32)
    w = np.empty((T, n_used), dtype=np.float32)
    rows = np.arange(T)
    for r in range(n_used):
        best = np.argmax(keys, axis=1)          # the first (lowest index) among equals
        ids[:, r] = best
        w[:, r] = weights[rows, best]
        keys[rows, best] = -np.inf
    return ids, w


def _normalised(w, norm, scale):
    ws = np.zeros(w.shape[0], dtype=np.float32)
    for r in range(w.shape[1]):
        ws = (ws + w[:, r]).astype(np.float32)
    ws = np.maximum(ws, np.float32(6.103515625e-5))
    out = (w / ws[:, None]).astype(np.float32) if norm else w
    return (out * np.float32(scale)).astype(np.float32) if scale != 1.0 else out


def moe_router(logits, n_used, x=None, w_shexp=None):
    """(ids, wts, sg) of the reference's softmax router (src/gpu_ops.hip:184-241): p = exp(l - max) * (1 / sum),
    selection on p, weights p / max(sum of the selected, 2^-14); sg = sigmoid(x . w_shexp) or None. fp32 operations
    one by one; the softmax sum and the dot product are carried in double."""
    l = np.asarray(logits, dtype=np.float32)
    ex = np.exp((l - l.max(axis=1, keepdims=True)).astype(np.float32)).astype(np.float32)
    inv = np.float32(1.0) / ex.astype(np.float64).sum(axis=1, keepdims=True).astype(np.float32)
    p = (ex * inv).astype(np.float32)
    ids, w = _top_rounds(p, p, n_used)
    sg = None
    if w_shexp is not None:
        d = (np.asarray(x, np.float64) * np.asarray(w_shexp, np.float64)).sum(axis=1).astype(np.float32)
        sg = (np.float32(1.0) / (np.float32(1.0) + np.exp(-d).astype(np.float32))).astype(np.float32)
    return ids, _normalised(w, True, 1.0), sg


def moe_router_sigmoid(logits, bias, n_used, norm, scale):
    """(ids, wts) of the reference's sigmoid router (src/gpu_ops.hip:794-824): keys sigmoid(l) + bias, weights
    sigmoid(l), normalised if norm, times scale."""
    l = np.asarray(logits, dtype=np.float32)
    p = (np.float32(1.0) / (np.float32(1.0) + np.exp(-l).astype(np.float32))).astype(np.float32)
    ids, w = _top_rounds((p + np.asarray(bias, np.float32)).astype(np.float32), p, n_used)
    return ids, _normalised(w, norm, scale)


def relu2(x):
    """max(x, 0)^2 (src/gpu_ops.hip:826-838)."""
    v = np.maximum(np.asarray(x, dtype=np.float32), np.float32(0.0))
    return (v * v).astype(np.float32)


def _sigmoid32(x):
    x = np.asarray(x, dtype=np.float32)
    return (np.float32(1.0) / (np.float32(1.0) + np.exp(-x).astype(np.float32))).astype(np.float32)


def _silu32(x):
    x = np.asarray(x, dtype=np.float32)
    return (x / (np.float32(1.0) + np.exp(-x).astype(np.float32))).astype(np.float32)


def hc_norm(res_in, cur, inject, w, hc, eps):
    """(res_out or None, y) of hc_norm (src/gpu_ops.hip:340-378): res [T][hc][n], cur [T][n] or None, inject [T][hc],
    w [hc][n]; fp32 operations one by one."""
    v = np.asarray(res_in, dtype=np.float32)
    T, _, n = v.shape
    out = None
    if cur is not None:
        wt = (np.float32(2.0) * _sigmoid32(np.asarray(inject, np.float32) * (np.float32(1.0) / np.float32(hc)))).astype(np.float32)
        v = (v + (np.asarray(cur, np.float32)[:, None, :] * wt[:, :, None]).astype(np.float32)).astype(np.float32)
        out = v
    inv = _row_inv_rms(v.reshape(T * hc, n), eps).reshape(T, hc, 1)
    return out, ((v * inv).astype(np.float32) * np.asarray(w, np.float32).reshape(1, hc, n)).astype(np.float32)


def hc_lowrank(lo, np_, hc):
    """SiLU(lo / hc) zero-padded to rows of np_ (src/gpu_ops.hip:380-394)."""
    lo = np.asarray(lo, dtype=np.float32)
    out = np.zeros((lo.shape[0], np_), dtype=np.float32)
    out[:, :lo.shape[1]] = _silu32((lo * (np.float32(1.0) / np.float32(hc))).astype(np.float32))
    return out


def hc_mix(xn, gate, hc):
    """Mean over the streams of xn * sigmoid(gate), streams added in order (src/gpu_ops.hip:396-409); [T][hc][n]."""
    xn, gate = np.asarray(xn, np.float32), np.asarray(gate, np.float32)
    acc = None
    for c in range(hc):
        p = (xn[:, c] * _sigmoid32(gate[:, c])).astype(np.float32)
        acc = p if acc is None else (acc + p).astype(np.float32)
    return (acc * (np.float32(1.0) / np.float32(hc))).astype(np.float32)


def ple_gate(key, value, res, wk, wq, wc, eps):
    """(gated, normed) of ple_gate (src/gpu_ops.hip:419-476): key / res [T][hc][n], value [T][n], gammas [hc][n]."""
    key, res, value = (np.asarray(a, np.float32) for a in (key, res, value))
    T, hc, n = key.shape
    wk, wq, wc = (np.asarray(a, np.float32).reshape(1, hc, n) for a in (wk, wq, wc))
    ik = _row_inv_rms(key.reshape(T * hc, n), eps).reshape(T, hc, 1)
    iq = _row_inv_rms(res.reshape(T * hc, n), eps).reshape(T, hc, 1)
    a = ((key * ik).astype(np.float32) * wk).astype(np.float32)
    b = ((res * iq).astype(np.float32) * wq).astype(np.float32)
    d = (a * b).astype(np.float32).astype(np.float64).sum(axis=2).astype(np.float32)
    s = (d * (np.float32(1.0) / np.sqrt(np.float32(n)))).astype(np.float32)
    mag = np.sqrt(np.maximum(np.abs(s), np.float32(1e-6))).astype(np.float32)
    g = _sigmoid32((np.sign(s).astype(np.float32) * mag).astype(np.float32))
    gated = (value[:, None, :] * g[:, :, None]).astype(np.float32)
    ig = _row_inv_rms(gated.reshape(T * hc, n), eps).reshape(T, hc, 1)
    return gated, ((gated * ig).astype(np.float32) * wc).astype(np.float32)


def mamba_gnorm(y, z, w, n_group, eps):
    """RMSNorm(y * SiLU(z)) * w per group of d_inner / n_group values (src/gpu_ops.hip:762-792)."""
    y, z, w = (np.asarray(a, np.float32) for a in (y, z, w))
    T, d = y.shape
    v = (y * _silu32(z)).astype(np.float32).reshape(T * n_group, d // n_group)
    return ((v * _row_inv_rms(v, eps)).astype(np.float32).reshape(T, d) * w).astype(np.float32)


def mamba_conv(zx, x_off, conv_state, w, bias, conv_dim, d_conv):
    """(out [T][conv_dim], new conv_state [conv_dim][d_conv - 1]) of mamba_conv / mamba_conv_state
    (src/gpu_ops.hip:702-728): window oldest first, products added one by one from 0, + bias, SiLU."""
    zx, w, bias = np.asarray(zx, np.float32), np.asarray(w, np.float32), np.asarray(bias, np.float32)
    st = np.asarray(conv_state, np.float32)
    T, ns = zx.shape[0], d_conv - 1
    x = np.concatenate([st.T, zx[:, x_off:x_off + conv_dim]], axis=0)          # rows: ns before the batch, then the batch
    s = np.zeros((T, conv_dim), np.float32)
    for k in range(d_conv):
        s = (s + (x[k:k + T] * w[:, k][None, :]).astype(np.float32)).astype(np.float32)
    return _silu32((s + bias[None, :]).astype(np.float32)), np.ascontiguousarray(x[T:T + ns].T)


def ple_conv(normed, gated, res, state, w_f16_bits, K, dil, n_mid=0):
    """(res, new state, mid states) of ple_conv (src/gpu_ops.hip:480-512): normed / gated / res [T][m], state
    [(K - 1) dil][m], w fp16 bit patterns [m][K]."""
    normed, gated, res, state = (np.asarray(a, np.float32) for a in (normed, gated, res, state))
    w = f16_to_f32(np.asarray(w_f16_bits, np.uint16)).reshape(-1, K)
    T, m = normed.shape
    H = (K - 1) * dil
    x = np.concatenate([state.reshape(H, m), normed], axis=0)
    acc = None
    for k in range(K):
        j0 = H - (K - 1 - k) * dil                                         # row of x that token 0 reads for tap k
        term = (x[j0:j0 + T] * w[:, k][None, :]).astype(np.float32)
        acc = term if acc is None else (acc + term).astype(np.float32)
    out = (res + (gated + _silu32(acc)).astype(np.float32)).astype(np.float32)
    mids = [np.ascontiguousarray(x[j + 1:j + 1 + H]) for j in range(min(n_mid, 3, max(T - 1, 0)))]
    return out, np.ascontiguousarray(x[T:T + H]), mids


def mamba_scan(state, xbc, zx, dt_off, dt_b, A, D, n_head, n_group):
    """(y [T][d_inner], new state) of mamba_scan (src/gpu_ops.hip:730-760): state [n_head][64][128]; per token
    dt = softplus(dt_t + dt_b) (ggml's: x itself above 20), dA = exp(dt A), s = s dA + B (x dt), y = sum_j s_j C_j + x D,
    the sum as 4 fused-multiply-add chains of 32 added pairwise ((0 + 1) + (2 + 3))."""
    s = np.array(state, dtype=np.float32).reshape(n_head, 64, 128)
    xbc, zx = np.asarray(xbc, np.float32), np.asarray(zx, np.float32)
    dt_b, A, D = (np.asarray(a, np.float32) for a in (dt_b, A, D))
    T, d_inner = xbc.shape[0], n_head * 64
    grp = np.arange(n_head) // (n_head // n_group)
    y = np.empty((T, d_inner), np.float32)
    for t in range(T):
        dv = (zx[t, dt_off:dt_off + n_head] + dt_b).astype(np.float32)
        sp = np.where(dv > 20, dv, np.log1p(np.exp(np.minimum(dv, 30).astype(np.float32)).astype(np.float32))).astype(np.float32)
        dA = np.exp((sp * A).astype(np.float32)).astype(np.float32)
        x = xbc[t, :d_inner].reshape(n_head, 64)
        xdt = (x * sp[:, None]).astype(np.float32)
        B = xbc[t, d_inner:d_inner + n_group * 128].reshape(n_group, 128)[grp]
        Cm = xbc[t, d_inner + n_group * 128:].reshape(n_group, 128)[grp]
        s = ((s * dA[:, None, None]).astype(np.float32) + (B[:, None, :] * xdt[:, :, None]).astype(np.float32)).astype(np.float32)
        q = np.zeros((n_head, 64, 4), np.float32)
        for j in range(32):                                               # fmaf chains: exact product, one rounding
            q = (s.reshape(n_head, 64, 4, 32)[..., j].astype(np.float64) * Cm.reshape(n_head, 1, 4, 32)[..., j] + q).astype(np.float32)
        acc = ((q[..., 0] + q[..., 1]).astype(np.float32) + (q[..., 2] + q[..., 3]).astype(np.float32)).astype(np.float32)
        y[t] = (acc + (x * D[:, None]).astype(np.float32)).astype(np.float32).reshape(d_inner)
    return y, s


def moe_combine(down, wts, shared=None, sg=None, ids=None, exp_scale=None):
    """out [T][n] = sum_j wts[t][j] * down[t][j] in slot order (+ shared * sg, or + shared), fp32 operations one by one
    (src/gpu_ops.hip:245-264): with exp_scale each term is (d * exp_scale[ids[t][j]]) * w; wts None: weight 1."""
    down = np.asarray(down, dtype=np.float32)
    T, n_used, n = down.shape
    acc = None
    for j in range(n_used):
        v = down[:, j, :]
        if wts is not None:
            w = np.asarray(wts, np.float32)[:, j:j + 1]
            if exp_scale is not None:
                es = np.asarray(exp_scale, np.float32)[np.asarray(ids)[:, j]][:, None]
                v = ((v * es).astype(np.float32) * w).astype(np.float32)
            else:
                v = (w * v).astype(np.float32)
        acc = v if acc is None else (acc + v).astype(np.float32)
    if shared is not None:
        sh = np.asarray(shared, np.float32)
        if sg is not None and wts is not None:
            sh = (sh * np.asarray(sg, np.float32)[:, None]).astype(np.float32)
        acc = (acc + sh).astype(np.float32)
    return acc


def gemma_ffn_post(x, mlp, down, wts, ids, exp_scale, w1, w2, w_post, scale, w_next, eps):
    """(x_out, y) of the reference's gemma_ffn_post kernel (src/gpu_ops.hip:608-655), fp32 operations one by one:
    c = moe_combine; h = RMSNorm(mlp) * w1 + RMSNorm(c) * w2; x_out = (x + RMSNorm(h) * w_post) * scale;
    y = RMSNorm(x_out) * w_next."""
    f = lambda t: np.asarray(t, dtype=np.float32)
    x, mlp, w1, w2, w_post, w_next = map(f, (x, mlp, w1, w2, w_post, w_next))
    c = moe_combine(down, wts, ids=ids, exp_scale=exp_scale)
    h = ((mlp * _row_inv_rms(mlp, eps)) * w1).astype(np.float32)
    h = (h + (c * _row_inv_rms(c, eps)) * w2).astype(np.float32)
    s = np.float32(1.0 if scale is None else scale)
    x_out = ((x + (h * _row_inv_rms(h, eps)) * w_post) * s).astype(np.float32)
    return x_out, ((x_out * _row_inv_rms(x_out, eps)) * w_next).astype(np.float32)


def geglu(gate, up):
    """GELU_tanh(g) * u (src/gpu_ops.hip:665-667): 0.5 x (1 + tanh(0.7978845608 x (1 + 0.044715 x x))) * u, fp32
    products left to right, tanh correctly rounded."""
    x, u = np.asarray(gate, dtype=np.float32), np.asarray(up, dtype=np.float32)
    c1, c2, one, half = np.float32(0.7978845608028654), np.float32(0.044715), np.float32(1.0), np.float32(0.5)
    inner = ((c1 * x) * (one + (c2 * x) * x)).astype(np.float32)
    t = np.tanh(inner.astype(np.float64)).astype(np.float32)
    return (((half * x) * (one + t)) * u).astype(np.float32)


def softcap(x, cap):
    """cap * tanh(x / cap) (src/gpu_ops.hip:673-677)."""
    x, cap = np.asarray(x, dtype=np.float32), np.float32(cap)
    return (cap * np.tanh((x / cap).astype(np.float64)).astype(np.float32)).astype(np.float32)


class Lcg:
    """The reference tests' generator (tests/layernorm_verify.cpp:29-33)."""

    def __init__(self, seed):
        self.state = C.c_uint32(seed)

    def rnd(self, lo, hi):
        return port().orc_lcg(C.byref(self.state), lo, hi)

    def next_u32(self):
        self.state = C.c_uint32((self.state.value * 1664525 + 1013904223) & 0xFFFFFFFF)
        return self.state.value
