"""Writes small GGUF files for the tests (the public container layout, version 3)."""
import struct

import numpy as np

T_U16, T_U32, T_F32, T_STR, T_ARR = 2, 4, 6, 8, 9


def _s(b):
    b = b.encode() if isinstance(b, str) else b
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, kv, tensors, alignment=32, version=3):
    """kv: list of (key, type, value); tensors: list of (name, ggml_type, ne (fastest first), bytes array)."""
    out = bytearray(struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kv)))
    for key, t, v in kv:
        out += _s(key) + struct.pack("<I", t)
        if t == T_U32:
            out += struct.pack("<I", v)
        elif t == T_U16:
            out += struct.pack("<H", v)
        elif t == T_F32:
            out += struct.pack("<f", v)
        elif t == T_STR:
            out += _s(v)
        elif t == T_ARR:        # v = (elem_type, list)
            et, items = v
            out += struct.pack("<IQ", et, len(items))
            for it in items:
                out += _s(it) if et == T_STR else struct.pack("<i", it)
    offs, off = [], 0
    for _, _, _, data in tensors:
        offs.append(off)
        off += (np.ascontiguousarray(data).nbytes + alignment - 1) // alignment * alignment
    for (name, typ, ne, _), o in zip(tensors, offs):
        out += _s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne)
        out += struct.pack("<IQ", typ, o)
    out += b"\0" * ((-len(out)) % alignment)
    data_off = len(out)
    for (_, _, _, data), o in zip(tensors, offs):
        assert len(out) == data_off + o
        b = np.ascontiguousarray(data).tobytes()
        out += b + b"\0" * ((-len(b)) % alignment)
    with open(path, "wb") as f:
        f.write(out)
    return data_off, offs
