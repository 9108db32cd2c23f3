"""Generates tests/golden/*.npz: inputs and outputs of the REFERENCE's own CPU functions for the layer-op path.

Run where the reference's source tree is present (it compiles src/qwen_ops.cpp and src/quant_types.cpp from there
into oracle/_ref/libref_cpu.so via oracle/Makefile):

    python tests/golden/make_golden.py

The fixtures pin the restatement in oracle/oracle_ops.c where the reference itself is absent. Inputs are seeded
(rocm_hip_b200.synth) and stored next to the outputs so the files stand alone.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from rocm_hip_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def main():
    O.build()
    R = O.ref()
    p = O.ptr

    # ---- qwen_rmsnorm (src/qwen_ops.cpp:8-13): hidden 1024 with gamma, head_dim 128 without, an odd width
    cases = {}
    for name, T, n, with_w, eps in (("h1024", 8, 1024, True, 1e-6), ("d128", 24, 128, False, 1e-6),
                                     ("n17", 8, 17, True, 1e-5), ("n5120", 2, 5120, True, 1e-6)):
        x = synth.normal(0, "g.rms." + name, 0, T * n).reshape(T, n)
        w = synth.normal(0, "g.rmsw." + name, 0, n, 1.0, 0.1) if with_w else None
        y = np.empty_like(x)
        for t in range(T):
            R.ref_qwen_rmsnorm(p(x[t]), p(w), p(y[t]), n, eps)
        cases[name + "_x"], cases[name + "_y"], cases[name + "_eps"] = x, y, np.float32(eps)
        if with_w:
            cases[name + "_w"] = w
    np.savez_compressed(os.path.join(OUT, "rmsnorm.npz"), **cases)

    # ---- qwen_rope_neox (src/qwen_ops.cpp:15-24): full and partial rotary, small and very large positions
    cases = {}
    positions = np.array([0, 1, 17, 2499, 4095, 32767, 131072, 262143], dtype=np.int32)
    for name, D, n_rot, base in (("d128_full_1e6", 128, 128, 1e6), ("d256_rot64_1e7", 256, 64, 1e7),
                                  ("d64_full_1e4", 64, 64, 1e4)):
        v = synth.normal(0, "g.rope." + name, 0, positions.size * D).reshape(positions.size, D)
        out = v.copy()
        for r, pos in enumerate(positions):
            R.ref_qwen_rope_neox(p(out[r]), n_rot, int(pos), base)
        cases[name + "_x"], cases[name + "_y"] = v, out
    cases["positions"] = positions
    np.savez_compressed(os.path.join(OUT, "rope_neox.npz"), **cases)

    # ---- qwen_silu (src/qwen_ops.h:47): N(0,1) draws, a sweep, and the extremes
    g = np.concatenate([synth.normal(0, "g.silu", 0, 4096), np.linspace(-30, 30, 1201, dtype=np.float32),
                        np.array([-104.0, -88.5, -87.0, -20.0, -0.0, 0.0, 1e-30, 20.0, 88.0, 89.0, 1e4, -1e4],
                                 dtype=np.float32)])
    s = np.array([R.ref_qwen_silu(float(v)) for v in g], dtype=np.float32)
    np.savez_compressed(os.path.join(OUT, "silu.npz"), g=g, silu=s)

    # ---- qt_to_float for Q8_0 / Q4_0 (src/quant_types.cpp:78-91,181-189), incl. special fp16 scales
    cases = {}
    E, rows = 256, 48
    special = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0xFBFF, 0x3C00, 0x1234, 0x83FF], dtype=np.uint16)
    for name, qt, maker in (("q8_0", O.Q8_0, synth.q8_0_table), ("q4_0", O.Q4_0, synth.q4_0_table)):
        tab = maker(0, "g.tab." + name, rows, E).copy()
        bb = 34 if qt == O.Q8_0 else 18
        blocks = tab.reshape(-1, bb)
        blocks[: special.size, 0:2] = special.view(np.uint8).reshape(-1, 2)  # first blocks get the special scales
        out = np.empty((rows, E), dtype=np.float32)
        for r in range(rows):
            assert R.qt_to_float(qt, p(tab[r]), p(out[r]), E) == 0
        assert R.qt_row_size(qt, E) == tab.shape[1]
        cases[name + "_table"], cases[name + "_out"] = tab, out
    np.savez_compressed(os.path.join(OUT, "dequant.npz"), **cases)

    # ---- qt_to_float for the other row formats the gather decodes (src/quant_types.cpp:58-74,126-179,264-345):
    #      random payload bytes (every nibble / high-bit / 6-bit scale pattern occurs), finite fp16 scales of both
    #      signs, and in the first blocks the special fp16 scales of above
    cases = {}
    E, rows = 512, 12
    for qt in (O.F32, O.F16, O.BF16, O.Q4_1, O.Q5_0, O.Q5_1, O.Q4_K, O.Q5_K, O.Q6_K):
        tab = synth.gguf_table(0, "g.any.%d" % qt, qt, rows, E).copy()
        blk, bb, halves = synth.GGUF_BLOCKS[qt]
        if halves:
            blocks = tab.reshape(-1, bb)
            for off in halves:
                blocks[: special.size, off:off + 2] = special.view(np.uint8).reshape(-1, 2)
        out = np.empty((rows, E), dtype=np.float32)
        for r in range(rows):
            assert R.qt_to_float(qt, p(tab[r]), p(out[r]), E) == 0
        assert R.qt_row_size(qt, E) == tab.shape[1]
        cases["t%d_table" % qt], cases["t%d_out" % qt] = tab, out
    np.savez_compressed(os.path.join(OUT, "dequant_more.npz"), **cases)

    # ---- qt_fp16_to_fp32 over every fp16 bit pattern, qt_bf16_to_fp32 likewise (src/quant_types.cpp:16-48)
    h = np.arange(65536, dtype=np.uint32)
    f16 = np.array([R.qt_fp16_to_fp32(int(v)) for v in h], dtype=np.float32)
    b16 = np.array([R.qt_bf16_to_fp32(int(v)) for v in h], dtype=np.float32)
    np.savez_compressed(os.path.join(OUT, "half_tables.npz"), fp16_bits=f16.view(np.uint32), bf16_bits=b16.view(np.uint32))
    print("golden fixtures written to", OUT)


if __name__ == "__main__":
    main()
