"""ctypes binding of libb200_layer_ops.so, the C-ABI library declared in include/b200_layer_ops.h.

The library is the product; this module only declares its entry points to ctypes. There is no fallback: if the
shared object has not been built (``python -c "import __graft_entry__ as g; g.build()"`` or
``make -C rocm_hip_b200/csrc``) loading raises, and so does every op.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200_layer_ops.so")

cudaSuccess = 0
cudaErrorInvalidValue = 1
cudaErrorInvalidDeviceFunction = 98


class qmatvec_q8(C.Structure):
    """Layout of the reference's struct qmatvec_q8 (src/qmatvec.h:70-83): device pointers of the side outputs."""
    _fields_ = [
        ("q0", C.c_void_p), ("d0", C.c_void_p), ("qK", C.c_void_p), ("dK", C.c_void_p), ("bsK", C.c_void_p),
        ("s0", C.c_void_p), ("max_k", C.c_int), ("xh", C.c_void_p), ("xh_bf16", C.c_int),
    ]


_p, _i, _ll, _f, _sz = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_size_t


class b200_layer_sweep(C.Structure):
    """Layout of struct b200_layer_sweep (include/b200_layer_ops.h): host row pointers of a layer's op sequence."""
    _fields_ = [
        ("elem", _i), ("T", _ll), ("qtype", _i), ("table_dev", _p), ("row_bytes", _sz), ("vocab", _i), ("tokens", _p),
        ("E", _i), ("embd_scale", _f), ("w_attn_norm", _p), ("w_ffn_norm", _p), ("w_next_norm", _p), ("eps", _f),
        ("xn_attn", _p), ("qfull", _p), ("k", _p), ("q_out", _p), ("k_out", _p), ("q_norm", _p), ("k_norm", _p),
        ("n_q", _i), ("n_kv", _i), ("head_dim", _i), ("n_rot", _i), ("rot_pairs", _i), ("positions", _p), ("pos0", _i),
        ("freq_base", _f), ("gated", _i), ("qk_norm", _i), ("freq_factors", _p), ("attn_proj", _p), ("xn_ffn", _p),
        ("gate", _p), ("up", _p), ("FF", _i), ("act", _p), ("ffn_proj", _p), ("x_out", _p), ("xn_next", _p),
    ]


# name -> (restype, argtypes); every symbol include/b200_layer_ops.h declares
SIGNATURES = {
    "gpu_ops_init": (_i, [C.c_char_p]),
    "gpu_ops_free": (None, []),
    "gpu_add_rmsnorm": (_i, [_p, _p, _p, _p, _p, _i, _i, _f, C.POINTER(qmatvec_q8), _p]),
    "gpu_swiglu": (_i, [_p, _p, _p, _i, C.POINTER(qmatvec_q8), _p]),
    "gpu_moe_group": (_i, [_p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p]),
    "gpu_add_rmsnorm_bf16": (_i, [_p, _p, _p, _p, _p, _i, _ll, _f, _p]),
    "gpu_add_rmsnorm_f32": (_i, [_p, _p, _p, _p, _p, _i, _ll, _f, _p]),
    "gpu_swiglu_bf16": (_i, [_p, _p, _p, _ll, _p]),
    "gpu_swiglu_f32": (_i, [_p, _p, _p, _ll, _p]),
    "gpu_swiglu_rows": (_i, [_p, _p, _p, _ll, _i, _ll, _ll, _p]),
    "gpu_swiglu_rows_bf16": (_i, [_p, _p, _p, _ll, _i, _ll, _ll, _p]),
    "gpu_qk_norm_rope": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _ll, _f, _f, _i, _i, _p, _p]),
    "gpu_qk_norm_rope_bf16": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _ll, _f, _f, _i, _i, _p, _p]),
    "gpu_moe_group_scratch_ints": (_sz, [_i, _i, _i]),
    "gpu_moe_group_scratch": (_i, [_p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "gpu_hadamard_rot": (_i, [_p, _p, _ll, _i, _i, _p]),
    "gpu_hadamard_rot_bf16": (_i, [_p, _p, _ll, _i, _i, _p]),
    "gpu_kv_store_q_rot": (_i, [_p, _p, _i, _p, _i, _ll, _i, _i, _ll, _i, _i, _p]),
    "gpu_kv_store_q_rot_bf16": (_i, [_p, _p, _i, _p, _i, _ll, _i, _i, _ll, _i, _i, _p]),
    "gpu_add_normed": (_i, [_p, _p, _p, _p, _p, _i, _i, _f, _p]),
    "gpu_gemma_attn_post": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _f, _p]),
    "gpu_gemma_ffn_post": (_i, [_p] * 6 + [_i] + [_p] * 8 + [_i, _i, _f, _p]),
    "gpu_mamba_conv": (_i, [_p, _ll, _i, _p, _p, _p, _p, _i, _i, _i, _p]),
    "gpu_mamba_scan": (_i, [_p, _p, _p, _ll, _i, _p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "gpu_ple_conv": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p]),
    "gpu_hc_norm": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _f, _p, _p]),
    "gpu_hc_lowrank": (_i, [_p, _p, _i, _i, _i, _i, _p, _p]),
    "gpu_hc_mix": (_i, [_p, _p, _p, _i, _i, _i, _p, _p]),
    "gpu_ple_gate": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _f, _p]),
    "gpu_mtp_concat": (_i, [_p, _p, _p, _i, _i, _i, _p]),
    "gpu_mamba_gnorm": (_i, [_p, _p, _ll, _p, _p, _i, _i, _i, _f, _p, _p]),
    "gpu_moe_router": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _i]),
    "gpu_moe_router_sigmoid": (_i, [_p, _p, _p, _p, _i, _i, _i, _f, _i, _p]),
    "gpu_relu2": (_i, [_p, _p, _i, _i, _i, _p, _p]),
    "gpu_moe_combine": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "gpu_moe_combine_scaled": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "gpu_geglu": (_i, [_p, _p, _p, _i, _i, _i, _i, _p, _p]),
    "gpu_softcap": (_i, [_p, _i, _f, _p]),
    "gpu_rope_table": (_i, [_p, _i, _ll, _i, _i, _f, _p, _p, _p, _p]),
    "gpu_qk_norm_rope_tab": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _ll, _f, _i, _i, _p]),
    "gpu_qk_norm_rope_tab_bf16": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _ll, _f, _i, _i, _p]),
    "gpu_qk_norm_rope_tab_kv": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _ll, _i, _i, _i, _i, _p, _p, _p, _i, _ll, _f, _i, _i, _p]),
    "gpu_qk_norm_rope_tab_kv_bf16": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _ll, _i, _i, _i, _i, _p, _p, _p, _i, _ll, _f, _i, _i, _p]),
    "gpu_qk_norm_rope_kv": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _ll, _i, _i, _i, _i, _i, _p, _i, _ll, _f, _f, _i, _i, _p, _p]),
    "gpu_qk_norm_rope_kv_bf16": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _ll, _i, _i, _i, _i, _i, _p, _i, _ll, _f, _f, _i, _i, _p, _p]),
    "gpu_attn_prep_f16": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _ll, _i, _i, _i, _i, _i, _p, _i, _ll, _f, _f, _i, _i, _p, _p]),
    "gpu_attn_prep_f16_bf16": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _ll, _i, _i, _i, _i, _i, _p, _i, _ll, _f, _f, _i, _i, _p, _p]),
    "gpu_kv_store_f16": (_i, [_p, _p, _i, _p, _i, _ll, _i, _i, _ll, _p]),
    "gpu_kv_store_f16_bf16": (_i, [_p, _p, _i, _p, _i, _ll, _i, _i, _ll, _p]),
    "gpu_kv_store_q": (_i, [_p, _p, _i, _p, _i, _ll, _i, _i, _ll, _i, _p]),
    "gpu_kv_store_q_bf16": (_i, [_p, _p, _i, _p, _i, _ll, _i, _i, _ll, _i, _p]),
    "gpu_embed_rows": (_i, [_i, _p, _sz, _i, _p, _p, _i, _ll, _f, _p, _p]),
    "gpu_embed_rows_bf16": (_i, [_i, _p, _sz, _i, _p, _p, _i, _ll, _f, _p, _p]),
    "gpu_embed_rows_host_ids": (_i, [_i, _p, _sz, _i, _p, _p, _p, _i, _ll, _f, _p, _p]),
    "gpu_embed_rows_static_scratch": (_i, [_i, _p, _sz, _i, _p, _p, _i, _ll, _f, _p]),
    "gpu_rmsnorm_f16": (_i, [_p, _p, _p, _i, _i, _f, _p]),
    "gpu_rope_rotate_half_f16": (_i, [_p, _p, _p, _p, _i, _i, _p]),
    "b200_host_ctx_create": (_p, [_sz, _i]),
    "b200_host_ctx_destroy": (None, [_p]),
    "b200_host_add_rmsnorm": (_i, [_p, _i, _p, _p, _p, _p, _p, _i, _ll, _f]),
    "b200_host_swiglu": (_i, [_p, _i, _p, _p, _p, _ll, _i]),
    "b200_host_qk_norm_rope": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _ll, _f, _f, _i, _i, _p]),
    "b200_host_embed_rows": (_i, [_p, _i, _i, _p, _sz, _i, _p, _p, _i, _ll, _f]),
    "b200_host_group_create": (_p, [_i, _sz, _i]),
    "b200_host_group_destroy": (None, [_p]),
    "b200_host_group_size": (_i, [_p]),
    "b200_host_group_add_rmsnorm": (_i, [_p, _i, _p, _p, _p, _p, _p, _i, _ll, _f]),
    "b200_host_layer_sweep": (_i, [_p, C.POINTER(b200_layer_sweep)]),
    "b200_host_group_swiglu": (_i, [_p, _i, _p, _p, _p, _ll, _i]),
    "b200_host_group_qk_norm_rope": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _ll, _f, _f, _i, _i, _p]),
    "b200_host_group_embed_rows": (_i, [_p, _i, _i, _p, _sz, _i, _p, _p, _i, _ll, _f]),
    "b200_host_group_layer_sweep": (_i, [_p, _p, _p]),
    "b200_host_chunk_plan": (_i, [_ll, _ll, _i, C.POINTER(_ll), _i]),
    "b200_gguf_open": (_p, [C.c_char_p]),
    "b200_gguf_close": (None, [_p]),
    "b200_gguf_n_tensors": (_ll, [_p]),
    "b200_gguf_version": (C.c_uint, [_p]),
    "b200_gguf_alignment": (_sz, [_p]),
    "b200_gguf_data_offset": (_sz, [_p]),
    "b200_gguf_n_files": (_i, [_p]),
    "b200_gguf_tensor_file": (_i, [_p, _i]),
    "b200_gguf_find_tensor": (_i, [_p, C.c_char_p]),
    "b200_gguf_tensor_info": (_i, [_p, _i, C.POINTER(C.c_char_p), C.POINTER(_i), C.POINTER(_i), C.POINTER(_ll * 4),
                                   C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_p)]),
    "b200_gguf_kv_u32": (_i, [_p, C.c_char_p, C.POINTER(C.c_uint32)]),
    "b200_gguf_kv_f32": (_i, [_p, C.c_char_p, C.POINTER(_f)]),
    "b200_gguf_kv_str": (_ll, [_p, C.c_char_p, C.c_char_p, _sz]),
    "b200_gguf_upload_tensor": (_i, [_p, _i, C.POINTER(_p), _p]),
    "b200_gguf_free_tensor": (None, [_p]),
    "b200_launch_count": (C.c_ulonglong, []),
    "b200_build_arch": (C.c_char_p, []),
}

_lib = None


def load():
    """Loads the library once and returns the ctypes handle. Raises if it is missing or lacks a declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is not built: run `make -C rocm_hip_b200/csrc` (needs nvcc); there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
