"""This library's GGUF reader (b200_gguf_*) against the REFERENCE'S OWN reader (src/gguf_mmap.cpp, compiled unchanged
into oracle/_ref/libref_gguf.so by oracle/Makefile) on the same files: tensor table, types, extents, sizes, alignment,
data offsets and the bytes both hand out, for a single file and for a split model opened by its first file
(src/gguf_mmap.cpp:384-437). The reference's reader accepting the files also checks tests/gguf_writer.py. No GPU."""
import ctypes as C
import os

import numpy as np
import pytest

from gguf_writer import T_ARR, T_F32, T_STR, T_U16, T_U32, write_gguf
from rocm_hip_b200 import _lib, synth

REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_gguf.so")
pytestmark = pytest.mark.skipif(not os.path.exists(REF_SO), reason="the reference's reader is built only where its sources are")


def ref_lib():
    L = C.CDLL(REF_SO)
    p, ll, sz = C.c_void_p, C.c_longlong, C.c_size_t
    for name, res, args in (("gguf_mmap_open", p, [C.c_char_p]), ("gguf_mmap_close", None, [p]), ("gguf_n_tensors", ll, [p]),
                            ("gguf_tensor_name", C.c_char_p, [p, ll]), ("gguf_tensor_type", C.c_int, [p, ll]),
                            ("gguf_tensor_ne", C.POINTER(ll), [p, ll]), ("gguf_tensor_dims", C.c_uint8, [p, ll]),
                            ("qt_row_size", sz, [C.c_int, ll]), ("gguf_tensor_offset", C.c_uint64, [p, ll]),
                            ("gguf_tensor_nbytes", sz, [p, ll]), ("gguf_alignment", sz, [p]), ("gguf_data_offset", sz, [p]),
                            ("gguf_version", C.c_uint32, [p]), ("gguf_get_tensor_ptr", p, [p, C.c_char_p, C.POINTER(sz)]),
                            ("gguf_n_maps", C.c_int, [p]), ("gguf_tensor_split", C.c_int, [p, ll]),
                            ("gguf_embedding_length", ll, [p]), ("gguf_arch", C.c_char_p, [p])):
        getattr(L, name).restype, getattr(L, name).argtypes = res, args
    return L


def mine(lib, g, idx):
    name, typ, nd = C.c_char_p(), C.c_int(), C.c_int()
    ne = (C.c_longlong * 4)()
    rb, nb, data = C.c_size_t(), C.c_size_t(), C.c_void_p()
    assert lib.b200_gguf_tensor_info(g, idx, C.byref(name), C.byref(typ), C.byref(nd), C.byref(ne), C.byref(rb),
                                     C.byref(nb), C.byref(data)) == 0
    return name.value, typ.value, nd.value, list(ne), rb.value, nb.value, data.value


def same_tables(path):
    lib, R = _lib.load(), ref_lib()
    g, r = lib.b200_gguf_open(path.encode()), R.gguf_mmap_open(path.encode())
    assert g and r
    try:
        n = R.gguf_n_tensors(r)
        assert lib.b200_gguf_n_tensors(g) == n and lib.b200_gguf_version(g) == R.gguf_version(r)
        assert lib.b200_gguf_alignment(g) == R.gguf_alignment(r) and lib.b200_gguf_data_offset(g) == R.gguf_data_offset(r)
        assert lib.b200_gguf_n_files(g) == R.gguf_n_maps(r)
        for i in range(n):
            name, typ, nd, ne, rb, nb, data = mine(lib, g, i)
            assert name == R.gguf_tensor_name(r, i) and typ == R.gguf_tensor_type(r, i) and nd == R.gguf_tensor_dims(r, i)
            assert ne[:nd] == [R.gguf_tensor_ne(r, i)[d] for d in range(nd)]
            assert lib.b200_gguf_tensor_file(g, i) == R.gguf_tensor_split(r, i)
            assert lib.b200_gguf_find_tensor(g, name) == i
            if nb:                                      # a type this library sizes
                assert rb == R.qt_row_size(typ, ne[0]) and nb == R.gguf_tensor_nbytes(r, i)   # (the unpadded row: src/quant_types.cpp:641)
                sz = C.c_size_t()
                rp = R.gguf_get_tensor_ptr(r, name, C.byref(sz))
                assert rp and sz.value == nb
                a = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), (nb,))
                b = np.ctypeslib.as_array(C.cast(rp, C.POINTER(C.c_uint8)), (nb,))
                assert np.array_equal(a, b), name
        return n, R.gguf_embedding_length(r), R.gguf_arch(r)
    finally:
        lib.b200_gguf_close(g)
        R.gguf_mmap_close(r)


def some_tensors(seed, vocab, E, prefix=""):
    q8 = synth.q8_0_table(seed, "gr.q8", vocab, E)
    q4 = synth.q4_0_table(seed, "gr.q4", 40, 64)
    norm = synth.normal(seed, "gr.norm", 0, E, 1.0, 0.1)
    f16 = synth.normal(seed, "gr.f16", 0, 3 * 64).astype(np.float16)
    k6 = synth.randint(seed, "gr.k6", 0, 2 * 210, 0, 256).astype(np.uint8)
    return [(prefix + "token_embd.weight", 8, (E, vocab), q8), (prefix + "output_norm.weight", 0, (E,), norm),
            (prefix + "small.weight", 2, (64, 40), q4), (prefix + "half.weight", 1, (64, 3), f16),
            (prefix + "k6.weight", 14, (256, 2), k6)]


@pytest.mark.parametrize("alignment,version", [(32, 3), (64, 3), (128, 3), (4096, 3)])
def test_one_file(tmp_path, alignment, version):
    kv = [("general.architecture", T_STR, "qwen3"), ("general.alignment", T_U32, alignment),
          ("qwen3.embedding_length", T_U32, 256), ("qwen3.attention.layer_norm_rms_epsilon", T_F32, 1e-6),
          ("tokenizer.ggml.tokens", T_ARR, (T_STR, ["a", "bc", "def"])), ("tokenizer.ggml.token_type", T_ARR, (5, [1, 2, 3]))]
    path = str(tmp_path / "one.gguf")
    write_gguf(path, kv, some_tensors(0, 300, 256), alignment, version)
    n, emb, arch = same_tables(path)
    assert (n, emb, arch) == (5, 256, b"qwen3")


def test_split_model_opened_by_its_first_file(tmp_path):
    base = [("general.architecture", T_STR, "qwen3"), ("qwen3.embedding_length", T_U32, 128)]
    for i, align in enumerate((32, 64, 32)):
        kv = base + [("general.alignment", T_U32, align), ("split.no", T_U16, i), ("split.count", T_U16, 3),
                     ("split.tensors.count", T_U32, 15)]
        write_gguf(str(tmp_path / f"m-{i + 1:05d}-of-00003.gguf"), kv, some_tensors(i, 100 + i, 128, prefix=f"p{i}."), align)
    n, emb, _ = same_tables(str(tmp_path / "m-00001-of-00003.gguf"))
    assert (n, emb) == (15, 128)
    lib, R = _lib.load(), ref_lib()
    # a later file cannot be the entry, a missing part or a part that names itself wrongly refuses the model: both readers
    for bad in ("m-00002-of-00003.gguf",):
        p = str(tmp_path / bad).encode()
        assert not lib.b200_gguf_open(p) and not R.gguf_mmap_open(p)
    os.rename(str(tmp_path / "m-00003-of-00003.gguf"), str(tmp_path / "gone.gguf"))
    p = str(tmp_path / "m-00001-of-00003.gguf").encode()
    assert not lib.b200_gguf_open(p) and not R.gguf_mmap_open(p)
    os.link(str(tmp_path / "m-00002-of-00003.gguf"), str(tmp_path / "m-00003-of-00003.gguf"))   # says split.no 1, not 2
    assert not lib.b200_gguf_open(p) and not R.gguf_mmap_open(p)
