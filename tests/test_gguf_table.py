"""The GGUF tensor-table reader (b200_gguf_*) on files written by tests/gguf_writer.py: header, metadata of every
value kind (skipped or read), tensor infos, alignment, data pointers; malformed files are refused. No GPU needed."""
import ctypes as C
import os

import struct

import numpy as np
import pytest

from gguf_writer import T_ARR, T_F32, T_STR, T_U16, T_U32, write_gguf
from rocm_hip_b200 import _lib, synth


def info(lib, g, idx):
    name, typ, nd = C.c_char_p(), C.c_int(), C.c_int()
    ne = (C.c_longlong * 4)()
    rb, nb, data = C.c_size_t(), C.c_size_t(), C.c_void_p()
    assert lib.b200_gguf_tensor_info(g, idx, C.byref(name), C.byref(typ), C.byref(nd), C.byref(ne), C.byref(rb),
                                     C.byref(nb), C.byref(data)) == 0
    return name.value.decode(), typ.value, nd.value, list(ne), rb.value, nb.value, data.value


@pytest.mark.parametrize("alignment", [32, 64])
def test_reads_what_was_written(tmp_path, alignment):
    lib = _lib.load()
    vocab, E = 300, 256
    q8 = synth.q8_0_table(0, "gg.q8", vocab, E)
    q4 = synth.q4_0_table(0, "gg.q4", 40, 64)
    norm = synth.normal(0, "gg.norm", 0, E, 1.0, 0.1)
    kv = [("general.architecture", T_STR, "qwen3"), ("general.alignment", T_U32, alignment),
          ("qwen3.embedding_length", T_U32, E), ("qwen3.attention.layer_norm_rms_epsilon", T_F32, 1e-6),
          ("tokenizer.ggml.tokens", T_ARR, (T_STR, ["a", "bc", "def"])), ("tokenizer.ggml.token_type", T_ARR, (5, [1, 2, 3]))]
    tensors = [("token_embd.weight", 8, (E, vocab), q8), ("output_norm.weight", 0, (E,), norm),
               ("small.weight", 2, (64, 40), q4), ("odd.weight", 10, (256, 3), np.zeros(252, np.uint8))]
    path = str(tmp_path / "m.gguf")
    data_off, offs = write_gguf(path, kv, tensors, alignment)
    g = lib.b200_gguf_open(path.encode())
    assert g
    try:
        assert lib.b200_gguf_version(g) == 3 and lib.b200_gguf_n_tensors(g) == 4
        assert lib.b200_gguf_alignment(g) == alignment and lib.b200_gguf_data_offset(g) == data_off
        i = lib.b200_gguf_find_tensor(g, b"token_embd.weight")
        name, typ, nd, ne, rb, nb, data = info(lib, g, i)
        assert (name, typ, nd, ne[:2], rb, nb) == ("token_embd.weight", 8, 2, [E, vocab], E // 32 * 34, q8.size)
        assert np.array_equal(np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), (nb,)), q8.ravel())
        _, typ, nd, ne, rb, nb, data = info(lib, g, lib.b200_gguf_find_tensor(g, b"output_norm.weight"))
        assert (typ, nd, ne[0], rb, nb) == (0, 1, E, 4 * E, 4 * E)
        assert np.array_equal(np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_float)), (E,)), norm)
        _, typ, _, ne, rb, nb, _ = info(lib, g, lib.b200_gguf_find_tensor(g, b"small.weight"))
        assert (typ, ne[:2], rb, nb) == (2, [64, 40], 36, q4.size)
        _, typ, _, _, rb, nb, data = info(lib, g, lib.b200_gguf_find_tensor(g, b"odd.weight"))
        assert typ == 10 and nb == 0 and data is None            # a type this library does not size
        assert lib.b200_gguf_find_tensor(g, b"nope") == -1
        u, f = C.c_uint32(), C.c_float()
        assert lib.b200_gguf_kv_u32(g, b"qwen3.embedding_length", C.byref(u)) == 0 and u.value == E
        assert lib.b200_gguf_kv_f32(g, b"qwen3.attention.layer_norm_rms_epsilon", C.byref(f)) == 0
        assert abs(f.value - 1e-6) < 1e-12
        assert lib.b200_gguf_kv_u32(g, b"general.architecture", C.byref(u)) == -1
        buf = C.create_string_buffer(32)
        assert lib.b200_gguf_kv_str(g, b"general.architecture", buf, 32) == 5 and buf.value == b"qwen3"
    finally:
        lib.b200_gguf_close(g)


def test_malformed_files_are_refused(tmp_path):
    lib = _lib.load()
    q8 = synth.q8_0_table(0, "gg.q8", 16, 64)
    path = str(tmp_path / "ok.gguf")
    write_gguf(path, [("general.alignment", T_U32, 32)], [("token_embd.weight", 8, (64, 16), q8)])
    raw = open(path, "rb").read()
    g = lib.b200_gguf_open(path.encode())
    assert g
    lib.b200_gguf_close(g)
    cases = {"magic": b"GGUX" + raw[4:], "version": raw[:4] + (9).to_bytes(4, "little") + raw[8:],
             "truncated_header": raw[:40], "truncated_data": raw[:-200], "empty": b"",
             "huge_count": raw[:8] + (2**40).to_bytes(8, "little") + raw[16:]}
    # extents whose byte count wraps around 2^64: 4 * ne0 * ne1 = 2^64 + 4096 for F32 rows of 4 values. The wrapped size
    # (4096 bytes) would fit the file; the open must fail rather than report a 2^60-row tensor as present.
    path = str(tmp_path / "wrap_src.gguf")
    write_gguf(path, [], [("token_embd.weight", 0, (4, 256), np.zeros((256, 4), np.float32))])
    wrap = bytearray(open(path, "rb").read())
    at = wrap.index(struct.pack("<QQ", 4, 256))
    wrap[at + 8:at + 16] = struct.pack("<Q", 2**60 + 256)
    cases["extent_product_wraps"] = bytes(wrap)
    # a file that ends right after the key and type of general.alignment (no value bytes to read)
    head = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 17) + b"general.alignment" + struct.pack("<I", T_U32)
    cases["alignment_value_missing"] = head
    for name, data in cases.items():
        p = str(tmp_path / (name + ".gguf"))
        open(p, "wb").write(data)
        assert not lib.b200_gguf_open(p.encode()), name
    assert not lib.b200_gguf_open(str(tmp_path / "missing.gguf").encode())


@pytest.mark.gpu
@pytest.mark.parametrize("split", [False, True])
def test_upload_and_gather(tmp_path, ops, oracle, split):
    """File -> device table -> gpu_embed_rows: the rows decode to what the CPU decoder makes of the file's bytes; also
    with the table in the second file of a split model."""
    import torch
    lib = _lib.load()
    vocab, E, T = 1000, 1024, 500
    q8 = synth.q8_0_table(1, "gg.up", vocab, E)
    arch = ("general.architecture", T_STR, "qwen3")
    pad, table = ("pad.weight", 0, (7,), np.zeros(7, np.float32)), ("token_embd.weight", 8, (E, vocab), q8)
    if split:
        path = str(tmp_path / "up-00001-of-00002.gguf")
        write_gguf(path, [arch, ("split.no", T_U16, 0), ("split.count", T_U16, 2)], [pad])
        write_gguf(str(tmp_path / "up-00002-of-00002.gguf"),
                   [arch, ("general.alignment", T_U32, 64), ("split.no", T_U16, 1), ("split.count", T_U16, 2)],
                   [("other.weight", 0, (5,), np.ones(5, np.float32)), table], alignment=64)
    else:
        path = str(tmp_path / "up.gguf")
        write_gguf(path, [arch], [pad, table])
    g = lib.b200_gguf_open(path.encode())
    assert g
    try:
        i = lib.b200_gguf_find_tensor(g, b"token_embd.weight")
        assert lib.b200_gguf_n_files(g) == (2 if split else 1) and lib.b200_gguf_tensor_file(g, i) == (1 if split else 0)
        _, typ, _, ne, rb, nb, _ = info(lib, g, i)
        dptr = C.c_void_p()
        assert lib.b200_gguf_upload_tensor(g, i, C.byref(dptr), None) == 0 and dptr.value
        ids = synth.randint(1, "gg.ids", 0, T, 0, vocab).astype(np.int32)
        d_ids = torch.from_numpy(ids).cuda()
        out = torch.zeros(T, E, device="cuda")
        bad = torch.full((1,), 2**31 - 1, dtype=torch.int32, device="cuda")
        assert lib.gpu_embed_rows(typ, dptr, rb, int(ne[1]), C.c_void_p(d_ids.data_ptr()), C.c_void_p(out.data_ptr()),
                                  int(ne[0]), T, 1.0, C.c_void_p(bad.data_ptr()), None) == 0
        torch.cuda.synchronize()
        _, want = oracle.embed_rows(oracle.Q8_0, q8, q8.shape[1], vocab, ids, E)
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
        lib.b200_gguf_free_tensor(dptr)
    finally:
        lib.b200_gguf_close(g)
