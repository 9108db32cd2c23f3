"""Python mirror of the launchers of include/b200_layer_ops.h for callers that hold torch CUDA tensors.

Names, argument order and error behaviour follow the C launchers (which follow src/gpu_ops.h:20-29 of the
reference): each function returns nothing and raises ``LayerOpError`` carrying the cudaError_t the launcher
returned. Launches go to torch's current stream and never synchronise. Nothing here computes: every function is one
call into the shared library, and the import fails if the library is absent.
"""
import ctypes as C

import torch

from . import _lib

__all__ = [
    "LayerOpError", "gpu_ops_init", "gpu_ops_free", "gpu_add_rmsnorm", "gpu_swiglu", "gpu_swiglu_rows",
    "gpu_qk_norm_rope", "gpu_rope_table", "gpu_qk_norm_rope_tab", "gpu_qk_norm_rope_tab_kv", "gpu_qk_norm_rope_kv", "gpu_attn_prep_f16", "gpu_embed_rows", "gpu_moe_group", "gpu_moe_group_scratch_ints", "gpu_moe_max_tiles", "gpu_kv_store_f16", "gpu_kv_store_q", "gpu_hadamard_rot", "gpu_add_normed", "gpu_gemma_attn_post", "gpu_geglu", "gpu_softcap", "gpu_gemma_ffn_post", "gpu_moe_combine", "gpu_moe_router", "gpu_moe_router_sigmoid", "gpu_relu2", "gpu_mamba_conv", "gpu_mamba_scan", "gpu_ple_conv", "gpu_hc_norm", "gpu_hc_lowrank", "gpu_hc_mix", "gpu_ple_gate", "gpu_mtp_concat", "gpu_mamba_gnorm", "gpu_rmsnorm_f16", "gpu_rope_rotate_half_f16", "launch_count", "Q8Buffers",
    "QT_Q4_0", "QT_Q8_0", "QT_F32", "QT_F16", "QT_BF16", "QT_Q4_1", "QT_Q5_0", "QT_Q5_1", "QT_Q4_K", "QT_Q5_K", "QT_Q6_K",
    "QT_BLOCKS", "qt_row_size", "HostRows", "HostGroup",
]

QT_Q4_0 = 2  # ggml type ids, src/quant_types.h:19-27 of the reference
QT_Q8_0 = 8
QT_F32, QT_F16, QT_Q4_1, QT_Q5_0, QT_Q5_1, QT_Q4_K, QT_Q5_K, QT_Q6_K, QT_BF16 = 0, 1, 3, 6, 7, 12, 13, 14, 30
# (values per block, bytes per block) of the row formats gpu_embed_rows decodes (src/quant_types.cpp:583-598)
QT_BLOCKS = {QT_F32: (1, 4), QT_F16: (1, 2), QT_BF16: (1, 2), QT_Q4_0: (32, 18), QT_Q4_1: (32, 20), QT_Q5_0: (32, 22),
             QT_Q5_1: (32, 24), QT_Q8_0: (32, 34), QT_Q4_K: (256, 144), QT_Q5_K: (256, 176), QT_Q6_K: (256, 210)}


def qt_row_size(qtype, ne0):
    """Bytes of one table row of ne0 values (src/quant_types.cpp:635-639); 0 if ne0 is not whole blocks."""
    blk, bb = QT_BLOCKS.get(qtype, (1, 0))
    return 0 if ne0 % blk else ne0 // blk * bb


class LayerOpError(RuntimeError):
    def __init__(self, what, code):
        super().__init__(f"{what}: cudaError {code}")
        self.code = code


def _check(what, code):
    if code != 0:
        raise LayerOpError(what, code)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def gpu_ops_init(co_path="gpu_ops.co"):
    return _lib.load().gpu_ops_init(co_path.encode())


def gpu_ops_free():
    _lib.load().gpu_ops_free()


def launch_count():
    return int(_lib.load().b200_launch_count())


class Q8Buffers:
    """Device buffers of a qmatvec_q8 for vectors of up to max_k values (max_k % 256 == 0), as the reference's
    qmatvec_q8_bind lays them out field by field (src/qmatvec.h:70-83). int8=False: only the 16-bit copy."""

    def __init__(self, max_k, device, xh=None, int8=True):
        assert max_k % 256 == 0
        self.max_k = max_k
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=device)
        self.q0 = z(max_k, torch.int8) if int8 else None
        self.d0 = z(max_k // 32, torch.float32) if int8 else None
        self.qK = z(max_k, torch.int8) if int8 else None
        self.dK = z(max_k // 256, torch.float32) if int8 else None
        self.bsK = z(max_k // 16, torch.int32) if int8 else None
        self.s0 = z(max_k // 32, torch.int32) if int8 else None
        self.xh = z(max_k, torch.int16) if xh else None
        self.xh_bf16 = 1 if xh == "bf16" else 0

    def struct(self):
        g = lambda t: None if t is None else t.data_ptr()
        return _lib.qmatvec_q8(g(self.q0), g(self.d0), g(self.qK), g(self.dK), g(self.bsK), g(self.s0), self.max_k,
                               g(self.xh), self.xh_bf16)


def gpu_add_rmsnorm(x_in, add, x_out, w, y, n, T, eps, q8=None):
    """x_out = x_in + add; y = RMSNorm(x_out) * w. fp32 tensors take the reference-named launcher (with q8), bf16
    tensors gpu_add_rmsnorm_bf16."""
    lib = _lib.load()
    if x_in.dtype == torch.float32:
        q = C.byref(q8.struct()) if q8 is not None else None
        if q8 is None and T > 2**31 - 1:
            code = lib.gpu_add_rmsnorm_f32(_ptr(x_in), _ptr(add), _ptr(x_out), _ptr(w), _ptr(y), n, T, eps, _stream())
        else:
            code = lib.gpu_add_rmsnorm(_ptr(x_in), _ptr(add), _ptr(x_out), _ptr(w), _ptr(y), n, T, eps, q, _stream())
    elif x_in.dtype == torch.bfloat16:
        assert q8 is None
        code = lib.gpu_add_rmsnorm_bf16(_ptr(x_in), _ptr(add), _ptr(x_out), _ptr(w), _ptr(y), n, T, eps, _stream())
    else:
        raise TypeError(x_in.dtype)
    _check("gpu_add_rmsnorm", code)


def gpu_swiglu(g, u, out, n, q8=None):
    lib = _lib.load()
    if g.dtype == torch.float32:
        if q8 is None and n > 2**31 - 1:
            code = lib.gpu_swiglu_f32(_ptr(g), _ptr(u), _ptr(out), n, _stream())
        else:
            q = C.byref(q8.struct()) if q8 is not None else None
            code = lib.gpu_swiglu(_ptr(g), _ptr(u), _ptr(out), n, q, _stream())
    elif g.dtype == torch.bfloat16:
        assert q8 is None
        code = lib.gpu_swiglu_bf16(_ptr(g), _ptr(u), _ptr(out), n, _stream())
    else:
        raise TypeError(g.dtype)
    _check("gpu_swiglu", code)


def gpu_swiglu_rows(gate, up, out, rows, h, gate_stride, up_stride):
    lib = _lib.load()
    fn = lib.gpu_swiglu_rows if gate.dtype == torch.float32 else lib.gpu_swiglu_rows_bf16
    _check("gpu_swiglu_rows", fn(_ptr(gate), _ptr(up), _ptr(out), rows, h, gate_stride, up_stride, _stream()))


def gpu_add_normed(base, a, w, scale, out, n, T, eps):
    """out = (base + RMSNorm(a) * w) * (scale[0] if scale is not None else 1) (src/gpu_ops.h:52)."""
    _check("gpu_add_normed", _lib.load().gpu_add_normed(_ptr(base), _ptr(a), _ptr(w), _ptr(scale), _ptr(out), n, T, eps,
                                                        _stream()))


def gpu_gemma_attn_post(x, a, w_a, x_out, w1, y1, w2, y2, n, T, eps, q8=None):
    """x_out = x + RMSNorm(a) * w_a; y1 = RMSNorm(x_out) * w1; y2 = RMSNorm(x_out) * w2 if w2 (src/gpu_ops.h:59)."""
    q = C.byref(q8.struct()) if q8 is not None else None
    _check("gpu_gemma_attn_post", _lib.load().gpu_gemma_attn_post(
        _ptr(x), _ptr(a), _ptr(w_a), _ptr(x_out), _ptr(w1), _ptr(y1), q, _ptr(w2), _ptr(y2), n, T, eps, _stream()))


def gpu_gemma_ffn_post(x, mlp, down, wts, ids, exp_scale, n_used, w1, w2, w_post, scale, x_out, w_next, y, n, T, eps,
                       q8=None):
    """The FFN epilogue of a Gemma-4 layer (src/gpu_ops.h:62): experts combined, two norms added, residual, scale,
    the next norm."""
    q = C.byref(q8.struct()) if q8 is not None else None
    _check("gpu_gemma_ffn_post", _lib.load().gpu_gemma_ffn_post(
        _ptr(x), _ptr(mlp), _ptr(down), _ptr(wts), _ptr(ids), _ptr(exp_scale), n_used, _ptr(w1), _ptr(w2), _ptr(w_post),
        _ptr(scale), _ptr(x_out), _ptr(w_next), _ptr(y), q, n, T, eps, _stream()))


def _q8arg(q8):
    return C.byref(q8.struct()) if q8 is not None else None


def gpu_mamba_conv(zx, ld, x_off, conv_state, w, bias, out, conv_dim, d_conv, T):
    """Mamba-2 causal conv1d + bias + SiLU, conv state advanced (src/gpu_ops.h:112)."""
    _check("gpu_mamba_conv", _lib.load().gpu_mamba_conv(_ptr(zx), ld, x_off, _ptr(conv_state), _ptr(w), _ptr(bias), _ptr(out),
                                                        conv_dim, d_conv, T, _stream()))


def gpu_mamba_scan(state, xbc, zx, ld, dt_off, dt_b, A, D, y, n_head, d_inner, n_group, T):
    """Mamba-2 selective scan (src/gpu_ops.h:114)."""
    _check("gpu_mamba_scan", _lib.load().gpu_mamba_scan(_ptr(state), _ptr(xbc), _ptr(zx), ld, dt_off, _ptr(dt_b), _ptr(A),
                                                        _ptr(D), _ptr(y), n_head, d_inner, n_group, T, _stream()))


def gpu_ple_conv(normed, gated, res, state, w, m, T, K, dil, state_mid=None):
    """PLE dilated causal depthwise conv (src/gpu_ops.h:97-101). w: float16 CUDA tensor [m][K]; state_mid: up to three
    CUDA tensors (or None entries) that receive the states after the first tokens."""
    mid = None
    if state_mid is not None:
        arr = (C.c_void_p * 3)(*[(t.data_ptr() if t is not None else None) for t in (list(state_mid) + [None] * 3)[:3]])
        mid = C.cast(arr, C.c_void_p)
    _check("gpu_ple_conv", _lib.load().gpu_ple_conv(_ptr(normed), _ptr(gated), _ptr(res), _ptr(state), _ptr(w), m, T, K, dil,
                                                    mid, _stream()))


def gpu_hc_norm(res_in, res_out, cur, inject, w, y, n, hc, T, eps, q8=None):
    """Hyper-connection combine + per-stream RMSNorm (src/gpu_ops.h:80-85)."""
    _check("gpu_hc_norm", _lib.load().gpu_hc_norm(_ptr(res_in), _ptr(res_out), _ptr(cur), _ptr(inject), _ptr(w), _ptr(y), n,
                                                  hc, T, eps, _q8arg(q8), _stream()))


def gpu_hc_lowrank(lo, out, n, np_, T, hc, q8=None):
    """out [T][np_] = SiLU(lo / hc), zero-padded (src/gpu_ops.h:86-89)."""
    _check("gpu_hc_lowrank", _lib.load().gpu_hc_lowrank(_ptr(lo), _ptr(out), n, np_, T, hc, _q8arg(q8), _stream()))


def gpu_hc_mix(xn, gate, out, n, hc, T, q8=None):
    """out[t] = mean over streams of xn * sigmoid(gate) (src/gpu_ops.h:90-92)."""
    _check("gpu_hc_mix", _lib.load().gpu_hc_mix(_ptr(xn), _ptr(gate), _ptr(out), n, hc, T, _q8arg(q8), _stream()))


def gpu_ple_gate(key, value, res, wk, wq, wc, gated, normed, n, hc, T, eps):
    """PLE gate (src/gpu_ops.h:93-96)."""
    _check("gpu_ple_gate", _lib.load().gpu_ple_gate(_ptr(key), _ptr(value), _ptr(res), _ptr(wk), _ptr(wq), _ptr(wc),
                                                    _ptr(gated), _ptr(normed), n, hc, T, eps, _stream()))


def gpu_mtp_concat(e, h, out, n, hc, T):
    """out [T][hc][2 n] = [e[t] | h[t][c]] (src/gpu_ops.h:103-105)."""
    _check("gpu_mtp_concat", _lib.load().gpu_mtp_concat(_ptr(e), _ptr(h), _ptr(out), n, hc, T, _stream()))


def gpu_mamba_gnorm(y, zx, ld, w, out, d_inner, n_group, T, eps, q8=None):
    """out = RMSNorm(y * SiLU(z)) * w per group (src/gpu_ops.h:117)."""
    _check("gpu_mamba_gnorm", _lib.load().gpu_mamba_gnorm(_ptr(y), _ptr(zx), ld, _ptr(w), _ptr(out), d_inner, n_group, T, eps,
                                                          _q8arg(q8), _stream()))


def gpu_moe_router(logits, x, w_shexp, ids, wts, sg, n_expert, n_used, n, T, ids_stride=0):
    """Softmax router (src/gpu_ops.h:30-37): ids / wts [T][n_used], optional shared-expert gate sg [T]."""
    _check("gpu_moe_router", _lib.load().gpu_moe_router(_ptr(logits), _ptr(x), _ptr(w_shexp), _ptr(ids), _ptr(wts), _ptr(sg),
                                                        n_expert, n_used, n, T, _stream(), ids_stride))


def gpu_moe_router_sigmoid(logits, bias, ids, wts, n_expert, n_used, norm, scale, T):
    """Sigmoid router (src/gpu_ops.h:119-123)."""
    _check("gpu_moe_router_sigmoid", _lib.load().gpu_moe_router_sigmoid(_ptr(logits), _ptr(bias), _ptr(ids), _ptr(wts),
                                                                        n_expert, n_used, norm, scale, T, _stream()))


def gpu_relu2(x, out, rows, h, stride, q8=None):
    """out [rows][h] = max(x, 0)^2 on strided rows (src/gpu_ops.h:124)."""
    q = C.byref(q8.struct()) if q8 is not None else None
    _check("gpu_relu2", _lib.load().gpu_relu2(_ptr(x), _ptr(out), rows, h, stride, q, _stream()))


def gpu_moe_combine(down, wts, shared, sg, out, n_used, n, T, ids=None, exp_scale=None):
    """out [T][n] = sum_j wts[t][j] * down[t][j] (+ sg[t] * shared[t]); with exp_scale, each expert's output scaled by
    exp_scale[ids[t][j]] first (src/gpu_ops.h:40-46)."""
    lib = _lib.load()
    if ids is None and exp_scale is None:
        code = lib.gpu_moe_combine(_ptr(down), _ptr(wts), _ptr(shared), _ptr(sg), _ptr(out), n_used, n, T, _stream())
    else:
        code = lib.gpu_moe_combine_scaled(_ptr(down), _ptr(wts), _ptr(shared), _ptr(sg), _ptr(ids), _ptr(exp_scale),
                                          _ptr(out), n_used, n, T, _stream())
    _check("gpu_moe_combine", code)


def gpu_geglu(gate, up, out, rows, h, gate_stride, up_stride, q8=None):
    """out [rows][h] = GELU_tanh(gate) * up on strided rows (src/gpu_ops.h:66)."""
    q = C.byref(q8.struct()) if q8 is not None else None
    _check("gpu_geglu", _lib.load().gpu_geglu(_ptr(gate), _ptr(up), _ptr(out), rows, h, gate_stride, up_stride, q,
                                              _stream()))


def gpu_softcap(x, n, cap):
    """x = cap * tanh(x / cap) in place (src/gpu_ops.h:68)."""
    _check("gpu_softcap", _lib.load().gpu_softcap(_ptr(x), n, cap, _stream()))


def gpu_kv_store_f16(src, cache, n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride):
    """Rows of src (fp32 or bf16) rounded to fp16 into the block-major KV cache `cache` (float16 CUDA tensor)."""
    lib = _lib.load()
    fn = lib.gpu_kv_store_f16 if src.dtype == torch.float32 else lib.gpu_kv_store_f16_bf16
    _check("gpu_kv_store_f16", fn(_ptr(src), _ptr(cache), n_vals, _ptr(positions), pos0, T, kv_stride, kv_shift,
                                  kv_bstride, _stream()))


def gpu_kv_store_q(src, cache, n_vals, positions, pos0, T, kv_stride, kv_shift, kv_bstride, kv_quant, rot_block=0):
    """Rows of src (fp32 or bf16) quantised to Q8_0 (kv_quant 1) or Q4_0 (2) into the block-major KV cache `cache`
    (a CUDA tensor of any 16-bit or byte dtype; kv_stride / kv_bstride in 2-byte units); rot_block 64 / 128 / 256:
    rotated in blocks of that many values first."""
    lib = _lib.load()
    if rot_block:
        fn = lib.gpu_kv_store_q_rot if src.dtype == torch.float32 else lib.gpu_kv_store_q_rot_bf16
        code = fn(_ptr(src), _ptr(cache), n_vals, _ptr(positions), pos0, T, kv_stride, kv_shift, kv_bstride, kv_quant,
                  rot_block, _stream())
    else:
        fn = lib.gpu_kv_store_q if src.dtype == torch.float32 else lib.gpu_kv_store_q_bf16
        code = fn(_ptr(src), _ptr(cache), n_vals, _ptr(positions), pos0, T, kv_stride, kv_shift, kv_bstride, kv_quant,
                  _stream())
    _check("gpu_kv_store_q", code)


def gpu_hadamard_rot(x, out, rows, D, block):
    """Orthonormal Walsh-Hadamard transform of rows of D values in blocks of `block` (src/attention.hip:238-263)."""
    lib = _lib.load()
    fn = lib.gpu_hadamard_rot if x.dtype == torch.float32 else lib.gpu_hadamard_rot_bf16
    _check("gpu_hadamard_rot", fn(_ptr(x), _ptr(out), rows, D, block, _stream()))


def gpu_moe_max_tiles(T, n_used, n_expert, tile):
    """Entries tile_e / tile_start / tile_n need (src/gpu_ops.h:68-71)."""
    n = T * n_used
    return min(n, n_expert + n // tile)


def gpu_moe_group(ids, T, n_used, n_expert, tile, tok_rows, pair_rows, n_tiles, tile_e, tile_start, tile_n, scratch=None):
    """Group the (token, slot) entries of ids [T][n_used] (int32) by expert; all arguments int32 CUDA tensors.
    scratch: an int32 CUDA tensor of gpu_moe_group_scratch_ints(...) entries to use instead of the library's own."""
    lib = _lib.load()
    if scratch is None:
        code = lib.gpu_moe_group(_ptr(ids), T, n_used, n_expert, tile, _ptr(tok_rows), _ptr(pair_rows), _ptr(n_tiles),
                                 _ptr(tile_e), _ptr(tile_start), _ptr(tile_n), _stream())
    else:
        code = lib.gpu_moe_group_scratch(_ptr(ids), T, n_used, n_expert, tile, _ptr(tok_rows), _ptr(pair_rows),
                                         _ptr(n_tiles), _ptr(tile_e), _ptr(tile_start), _ptr(tile_n), _ptr(scratch),
                                         scratch.numel(), _stream())
    _check("gpu_moe_group", code)


def gpu_moe_group_scratch_ints(T, n_used, n_expert):
    return int(_lib.load().gpu_moe_group_scratch_ints(T, n_used, n_expert))


def gpu_qk_norm_rope(qfull, k, q_norm, k_norm, q_out, k_out, n_q, n_kv, head_dim, n_rot, rot_pairs, positions, pos0, T,
                     freq_base, eps, gated=0, qk_norm=1, freq_factors=None):
    lib = _lib.load()
    ref = qfull if qfull is not None else k
    fn = lib.gpu_qk_norm_rope if ref.dtype == torch.float32 else lib.gpu_qk_norm_rope_bf16
    _check("gpu_qk_norm_rope",
           fn(_ptr(qfull), _ptr(k), _ptr(q_norm), _ptr(k_norm), _ptr(q_out), _ptr(k_out), n_q, n_kv, head_dim, n_rot,
              rot_pairs, _ptr(positions), pos0, T, freq_base, eps, gated, qk_norm, _ptr(freq_factors), _stream()))


def gpu_rope_table(positions, pos0, T, n_rot, rot_pairs, freq_base, cos_tab, sin_tab, freq_factors=None):
    """cos / sin tables [T][n_rot / 2] (fp32 CUDA tensors) of the angles gpu_qk_norm_rope would form."""
    _check("gpu_rope_table",
           _lib.load().gpu_rope_table(_ptr(positions), pos0, T, n_rot, rot_pairs, freq_base, _ptr(freq_factors),
                                      _ptr(cos_tab), _ptr(sin_tab), _stream()))


def gpu_qk_norm_rope_tab(qfull, k, q_norm, k_norm, q_out, k_out, n_q, n_kv, head_dim, n_rot, cos_tab, sin_tab, T, eps,
                         gated=0, qk_norm=1):
    """gpu_qk_norm_rope with the angles' cos / sin read from the tables of gpu_rope_table."""
    lib = _lib.load()
    ref = qfull if qfull is not None else k
    fn = lib.gpu_qk_norm_rope_tab if ref.dtype == torch.float32 else lib.gpu_qk_norm_rope_tab_bf16
    _check("gpu_qk_norm_rope_tab",
           fn(_ptr(qfull), _ptr(k), _ptr(q_norm), _ptr(k_norm), _ptr(q_out), _ptr(k_out), n_q, n_kv, head_dim, n_rot,
              _ptr(cos_tab), _ptr(sin_tab), T, eps, gated, qk_norm, _stream()))


def gpu_qk_norm_rope_kv(qfull, k, q_norm, k_norm, q_out, k_cache, kv_stride, kv_shift, kv_bstride, n_q, n_kv, head_dim, n_rot,
                        rot_pairs, positions, pos0, T, freq_base, eps, gated=0, qk_norm=1, freq_factors=None):
    """gpu_qk_norm_rope with the K heads written, rounded to fp16, into the block-major KV cache `k_cache`."""
    lib = _lib.load()
    fn = lib.gpu_qk_norm_rope_kv if k.dtype == torch.float32 else lib.gpu_qk_norm_rope_kv_bf16
    _check("gpu_qk_norm_rope_kv",
           fn(_ptr(qfull), _ptr(k), _ptr(q_norm), _ptr(k_norm), _ptr(q_out), _ptr(k_cache), kv_stride, kv_shift, kv_bstride,
              n_q, n_kv, head_dim, n_rot, rot_pairs, _ptr(positions), pos0, T, freq_base, eps, gated, qk_norm,
              _ptr(freq_factors), _stream()))


def gpu_qk_norm_rope_tab_kv(qfull, k, q_norm, k_norm, q_out, k_cache, kv_stride, kv_shift, kv_bstride, n_q, n_kv, head_dim,
                            n_rot, cos_tab, sin_tab, positions, pos0, T, eps, gated=0, qk_norm=1):
    """gpu_qk_norm_rope_kv with the cos / sin read from the tables of gpu_rope_table; positions / pos0 still name the
    cache rows."""
    lib = _lib.load()
    fn = lib.gpu_qk_norm_rope_tab_kv if k.dtype == torch.float32 else lib.gpu_qk_norm_rope_tab_kv_bf16
    _check("gpu_qk_norm_rope_tab_kv",
           fn(_ptr(qfull), _ptr(k), _ptr(q_norm), _ptr(k_norm), _ptr(q_out), _ptr(k_cache), kv_stride, kv_shift, kv_bstride,
              n_q, n_kv, head_dim, n_rot, _ptr(cos_tab), _ptr(sin_tab), _ptr(positions), pos0, T, eps, gated, qk_norm,
              _stream()))


def gpu_attn_prep_f16(qfull, k, v, q_norm, k_norm, q_out, K, V, kv_stride, kv_shift, kv_bstride, n_q, n_kv, head_dim, n_rot,
                      rot_pairs, positions, pos0, T, freq_base, eps, gated=0, qk_norm=1, freq_factors=None):
    """q/k norm + RoPE with K into the FP16 cache, then the V rows into it (two launches)."""
    lib = _lib.load()
    fn = lib.gpu_attn_prep_f16 if k.dtype == torch.float32 else lib.gpu_attn_prep_f16_bf16
    _check("gpu_attn_prep_f16",
           fn(_ptr(qfull), _ptr(k), _ptr(v), _ptr(q_norm), _ptr(k_norm), _ptr(q_out), _ptr(K), _ptr(V), kv_stride, kv_shift,
              kv_bstride, n_q, n_kv, head_dim, n_rot, rot_pairs, _ptr(positions), pos0, T, freq_base, eps, gated, qk_norm,
              _ptr(freq_factors), _stream()))


def gpu_embed_rows(qtype, table, row_bytes, vocab, tokens, out, E, T, scale=1.0, bad_row=None):
    """Gather + dequantise. tokens: int32 CUDA tensor. bad_row: int32 CUDA tensor of one element holding INT_MAX (one
    is made when None). Returns the bad_row tensor; the caller reads it after synchronising."""
    lib = _lib.load()
    if bad_row is None:
        bad_row = torch.full((1,), 2**31 - 1, dtype=torch.int32, device=out.device)
    fn = lib.gpu_embed_rows if out.dtype == torch.float32 else lib.gpu_embed_rows_bf16
    _check("gpu_embed_rows",
           fn(qtype, _ptr(table), row_bytes, vocab, _ptr(tokens), _ptr(out), E, T, scale, _ptr(bad_row), _stream()))
    return bad_row


def gpu_rmsnorm_f16(x, gamma, y, n_tokens, n_embd, eps):
    _check("gpu_rmsnorm_f16",
           _lib.load().gpu_rmsnorm_f16(_ptr(x), _ptr(gamma), _ptr(y), n_tokens, n_embd, eps, _stream()))


def gpu_rope_rotate_half_f16(x, ctab, stab, y, n_rows, half_dim):
    _check("gpu_rope_rotate_half_f16",
           _lib.load().gpu_rope_rotate_half_f16(_ptr(x), _ptr(ctab), _ptr(stab), _ptr(y), n_rows, half_dim, _stream()))


class HostRows:
    """The host-buffer entry points (b200_host_*): rows in host memory (numpy arrays or CPU torch tensors, ideally
    page-locked) are streamed through the device in chunks. Calls are synchronous. The embedding table stays a CUDA
    tensor. One context per device and caller thread."""

    def __init__(self, slot_bytes=64 << 20, n_slots=4):
        self._lib = _lib.load()
        self._ctx = self._lib.b200_host_ctx_create(slot_bytes, n_slots)
        if not self._ctx:
            raise LayerOpError("b200_host_ctx_create", -1)

    def close(self):
        if self._ctx:
            self._lib.b200_host_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _h(a):
        if a is None:
            return None
        if isinstance(a, torch.Tensor):
            assert not a.is_cuda and a.is_contiguous()
            return C.c_void_p(a.data_ptr())
        assert a.flags["C_CONTIGUOUS"]
        return C.c_void_p(a.ctypes.data)

    @staticmethod
    def _elem(a):
        return a.element_size() if isinstance(a, torch.Tensor) else a.dtype.itemsize

    def add_rmsnorm(self, x_in, add, x_out, w, y, n, T, eps):
        h = self._h
        _check("b200_host_add_rmsnorm", self._lib.b200_host_add_rmsnorm(
            self._ctx, self._elem(x_in), h(x_in), h(add), h(x_out), h(w), h(y), n, T, eps))

    def swiglu(self, g, u, out, rows, width):
        h = self._h
        _check("b200_host_swiglu", self._lib.b200_host_swiglu(self._ctx, self._elem(g), h(g), h(u), h(out), rows, width))

    def qk_norm_rope(self, qfull, k, q_norm, k_norm, q_out, k_out, n_q, n_kv, head_dim, n_rot, rot_pairs, positions,
                     pos0, T, freq_base, eps, gated=0, qk_norm=1, freq_factors=None):
        h = self._h
        ref = qfull if qfull is not None else k
        _check("b200_host_qk_norm_rope", self._lib.b200_host_qk_norm_rope(
            self._ctx, self._elem(ref), h(qfull), h(k), h(q_norm), h(k_norm), h(q_out), h(k_out), n_q, n_kv, head_dim,
            n_rot, rot_pairs, h(positions), pos0, T, freq_base, eps, gated, qk_norm, h(freq_factors)))

    def embed_rows(self, qtype, table_dev, row_bytes, vocab, tokens, out, E, T, scale=1.0):
        h = self._h
        _check("b200_host_embed_rows", self._lib.b200_host_embed_rows(
            self._ctx, self._elem(out), qtype, _ptr(table_dev), row_bytes, vocab, h(tokens), h(out), E, T, scale))


    def layer_sweep(self, *, qtype, table_dev, row_bytes, vocab, tokens, E, w_attn_norm, w_ffn_norm, w_next_norm, eps,
                    xn_attn, qfull, k, q_out, k_out, q_norm, k_norm, n_q, n_kv, head_dim, n_rot, freq_base, attn_proj,
                    xn_ffn, gate, up, FF, act, ffn_proj, x_out, xn_next, T, rot_pairs=0, positions=None, pos0=0, gated=0,
                    qk_norm=1, freq_factors=None, embd_scale=1.0):
        """b200_host_layer_sweep: the layer's six ops in one call; rows in host memory, the residual stream stays on
        the device between the kernels of a chunk."""
        a = self._sweep_args(locals())
        _check("b200_host_layer_sweep", self._lib.b200_host_layer_sweep(self._ctx, C.byref(a)))

    def _sweep_args(self, kw):
        """The b200_layer_sweep structure from layer_sweep's arguments (table_dev may be None: a group passes its own)."""
        g = kw.get
        v = lambda a: self._h(a).value if a is not None else None
        (qtype, row_bytes, vocab, tokens, E, w_attn_norm, w_ffn_norm, w_next_norm, eps, xn_attn, qfull, k, q_out, k_out, q_norm,
         k_norm, n_q, n_kv, head_dim, n_rot, freq_base, attn_proj, xn_ffn, gate, up, FF, act, ffn_proj, x_out, xn_next, T,
         rot_pairs, positions, pos0, gated, qk_norm, freq_factors, embd_scale) = (g(n) for n in (
            "qtype", "row_bytes", "vocab", "tokens", "E", "w_attn_norm", "w_ffn_norm", "w_next_norm", "eps", "xn_attn", "qfull",
            "k", "q_out", "k_out", "q_norm", "k_norm", "n_q", "n_kv", "head_dim", "n_rot", "freq_base", "attn_proj", "xn_ffn",
            "gate", "up", "FF", "act", "ffn_proj", "x_out", "xn_next", "T", "rot_pairs", "positions", "pos0", "gated", "qk_norm",
            "freq_factors", "embd_scale"))
        table_dev = g("table_dev")
        return _lib.b200_layer_sweep(
            elem=self._elem(xn_attn), T=T, qtype=qtype, table_dev=table_dev.data_ptr() if table_dev is not None else None,
            row_bytes=row_bytes, vocab=vocab,
            tokens=v(tokens), E=E, embd_scale=embd_scale, w_attn_norm=v(w_attn_norm), w_ffn_norm=v(w_ffn_norm),
            w_next_norm=v(w_next_norm), eps=eps, xn_attn=v(xn_attn), qfull=v(qfull), k=v(k), q_out=v(q_out), k_out=v(k_out),
            q_norm=v(q_norm), k_norm=v(k_norm), n_q=n_q, n_kv=n_kv, head_dim=head_dim, n_rot=n_rot, rot_pairs=rot_pairs,
            positions=v(positions), pos0=pos0, freq_base=freq_base, gated=gated, qk_norm=qk_norm,
            freq_factors=v(freq_factors), attn_proj=v(attn_proj), xn_ffn=v(xn_ffn), gate=v(gate), up=v(up), FF=FF,
            act=v(act), ffn_proj=v(ffn_proj), x_out=v(x_out), xn_next=v(xn_next))


class HostGroup(HostRows):
    """The same host-buffer calls over several GPUs of one box from one process (b200_host_group_*): rows are cut into
    contiguous ranges, one per device, and one host thread per device streams its range. embed_rows takes one CUDA
    table per device, in device order."""

    def __init__(self, n_devices=0, slot_bytes=64 << 20, n_slots=4):
        self._lib = _lib.load()
        self._ctx = self._lib.b200_host_group_create(n_devices, slot_bytes, n_slots)
        if not self._ctx:
            raise LayerOpError("b200_host_group_create", -1)
        self.size = self._lib.b200_host_group_size(self._ctx)

    def close(self):
        if self._ctx:
            self._lib.b200_host_group_destroy(self._ctx)
            self._ctx = None

    def add_rmsnorm(self, x_in, add, x_out, w, y, n, T, eps):
        h = self._h
        _check("b200_host_group_add_rmsnorm", self._lib.b200_host_group_add_rmsnorm(
            self._ctx, self._elem(x_in), h(x_in), h(add), h(x_out), h(w), h(y), n, T, eps))

    def swiglu(self, g, u, out, rows, width):
        h = self._h
        _check("b200_host_group_swiglu",
               self._lib.b200_host_group_swiglu(self._ctx, self._elem(g), h(g), h(u), h(out), rows, width))

    def qk_norm_rope(self, qfull, k, q_norm, k_norm, q_out, k_out, n_q, n_kv, head_dim, n_rot, rot_pairs, positions,
                     pos0, T, freq_base, eps, gated=0, qk_norm=1, freq_factors=None):
        h = self._h
        ref = qfull if qfull is not None else k
        _check("b200_host_group_qk_norm_rope", self._lib.b200_host_group_qk_norm_rope(
            self._ctx, self._elem(ref), h(qfull), h(k), h(q_norm), h(k_norm), h(q_out), h(k_out), n_q, n_kv, head_dim,
            n_rot, rot_pairs, h(positions), pos0, T, freq_base, eps, gated, qk_norm, h(freq_factors)))

    def layer_sweep(self, *, tables_dev, **kw):
        """b200_host_group_layer_sweep: layer_sweep's arguments with one CUDA table per device instead of table_dev."""
        assert len(tables_dev) == self.size
        kw.setdefault("rot_pairs", 0), kw.setdefault("positions", None), kw.setdefault("pos0", 0), kw.setdefault("gated", 0)
        kw.setdefault("qk_norm", 1), kw.setdefault("freq_factors", None), kw.setdefault("embd_scale", 1.0)
        a = self._sweep_args(dict(kw, table_dev=None))
        ptrs = (C.c_void_p * self.size)(*[t.data_ptr() for t in tables_dev])
        _check("b200_host_group_layer_sweep", self._lib.b200_host_group_layer_sweep(self._ctx, C.byref(a), ptrs))

    def embed_rows(self, qtype, tables_dev, row_bytes, vocab, tokens, out, E, T, scale=1.0):
        h = self._h
        assert len(tables_dev) == self.size
        ptrs = (C.c_void_p * self.size)(*[t.data_ptr() for t in tables_dev])
        _check("b200_host_group_embed_rows", self._lib.b200_host_group_embed_rows(
            self._ctx, self._elem(out), qtype, ptrs, row_bytes, vocab, h(tokens), h(out), E, T, scale))
