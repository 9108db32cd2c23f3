"""Seeded synthetic tensors with the shapes and value distributions of the five benchmark configurations. They stand
in for real-model activations and GGUF tensors, which a benchmark box does not hold.

The generator is counter based: a value depends only on (seed, tensor name, element index), so a row shard can
produce its slice without the rest and a row has the same values whatever the shard layout.
"""
import zlib

import numpy as np

_M = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix(z):
    z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M
    return z ^ (z >> np.uint64(31))


def _key(seed, name):
    return np.uint64((seed * 0x100000001B3 + zlib.crc32(name.encode())) & 0xFFFFFFFFFFFFFFFF)


def bits(seed, name, start, count, stream=0):
    """count 64-bit words for elements start .. start+count-1 of tensor `name`."""
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + count, dtype=np.uint64)
        return _splitmix(_splitmix(idx ^ _key(seed, name)) + np.uint64(stream))


def uniform(seed, name, start, count, stream=0):
    """float64 in (0, 1)."""
    return ((bits(seed, name, start, count, stream) >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)


def normal(seed, name, start, count, mean=0.0, std=1.0):
    """float32 N(mean, std) by Box-Muller on two streams of the element's counter."""
    u1, u2 = uniform(seed, name, start, count, 0), uniform(seed, name, start, count, 1)
    return (mean + std * np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def randint(seed, name, start, count, lo, hi):
    """int64 uniform in [lo, hi)."""
    return lo + (bits(seed, name, start, count) % np.uint64(hi - lo)).astype(np.int64)


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def q8_0_table(seed, name, vocab, E, row0=0, rows=None):
    """Q8_0 rows [rows][E/32 * 34] uint8: per block an fp16 scale ~U(1e-3, 2e-2) and 32 int8 uniform in [-127, 127]."""
    rows = vocab - row0 if rows is None else rows
    nb = E // 32
    nblk = rows * nb
    b0 = row0 * nb
    d = (1e-3 + uniform(seed, name + ".d", b0, nblk) * (2e-2 - 1e-3)).astype(np.float16)
    q = (randint(seed, name + ".q", b0 * 32, nblk * 32, -127, 128)).astype(np.int8)
    out = np.empty((nblk, 34), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nblk, 2)
    out[:, 2:] = q.view(np.uint8).reshape(nblk, 32)
    return out.reshape(rows, nb * 34)


def q4_0_table(seed, name, vocab, E, row0=0, rows=None):
    """Q4_0 rows [rows][E/32 * 18] uint8: per block an fp16 scale ~U(1e-3, 2e-2) and 32 nibbles uniform in [0, 15]."""
    rows = vocab - row0 if rows is None else rows
    nb = E // 32
    nblk = rows * nb
    b0 = row0 * nb
    d = (1e-3 + uniform(seed, name + ".d", b0, nblk) * (2e-2 - 1e-3)).astype(np.float16)
    q = randint(seed, name + ".q", b0 * 16, nblk * 16, 0, 256).astype(np.uint8)
    out = np.empty((nblk, 18), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nblk, 2)
    out[:, 2:] = q.reshape(nblk, 16)
    return out.reshape(rows, nb * 18)


# ggml type id -> (values per block, bytes per block, byte offsets of the fp16 fields of a block)
GGUF_BLOCKS = {0: (1, 4, ()), 1: (1, 2, ()), 30: (1, 2, ()), 2: (32, 18, (0,)), 3: (32, 20, (0, 2)), 6: (32, 22, (0,)),
               7: (32, 24, (0, 2)), 8: (32, 34, (0,)), 12: (256, 144, (0, 2)), 13: (256, 176, (0, 2)), 14: (256, 210, (208,))}


def gguf_table(seed, name, qtype, rows, E):
    """A table of `rows` rows of E values in GGUF row format `qtype` (a ggml type id of GGUF_BLOCKS) as uint8
    [rows][row bytes]: every payload byte uniform in [0, 255], the fp16 scale / minimum fields finite values
    ~U(1e-3, 2e-2) with random sign; F32 / F16 / BF16 rows are N(0, 1) values in that format."""
    blk, bb, halves = GGUF_BLOCKS[qtype]
    assert E % blk == 0
    if blk == 1:
        v = normal(seed, name + ".v", 0, rows * E)
        if qtype == 0:
            return v.view(np.uint8).reshape(rows, E * 4).copy()
        if qtype == 1:
            return v.astype(np.float16).view(np.uint8).reshape(rows, E * 2).copy()
        return f32_to_bf16_bits(v).view(np.uint8).reshape(rows, E * 2).copy()
    nblk = rows * (E // blk)
    out = randint(seed, name + ".q", 0, nblk * bb, 0, 256).astype(np.uint8).reshape(nblk, bb)
    for k, off in enumerate(halves):
        d = (1e-3 + uniform(seed, name + ".d%d" % k, 0, nblk) * (2e-2 - 1e-3))
        d = (d * np.where(uniform(seed, name + ".s%d" % k, 0, nblk) < 0.25, -1.0, 1.0)).astype(np.float16)
        out[:, off:off + 2] = d.view(np.uint8).reshape(nblk, 2)
    return out.reshape(rows, (E // blk) * bb)


def moe_routing(seed, name, T, n_expert, n_used):
    """Per token n_used distinct experts drawn uniformly; returns (ids [T][n_used], order) where order lists the
    T * n_used (token, slot) rows sorted by expert id, stable, as an expert-grouping pass would."""
    keys = uniform(seed, name, 0, T * n_expert).reshape(T, n_expert)
    ids = np.argsort(keys, axis=1, kind="stable")[:, :n_used].astype(np.int32)
    order = np.argsort(ids.ravel(), kind="stable")
    return ids, order


# The five benchmark configurations (row counts and widths of the reference's model shapes)
CONFIGS = {
    "c1_qwen3_0p6b_fp32": dict(dtype="f32", T=2427, E=1024, n_q=16, n_kv=8, D=128, n_rot=128, theta=1e6, FF=3072,
                               qtype=8, vocab=151936, eps=1e-6, positions="range"),
    "c2_decode_bf16": dict(dtype="bf16", T=64, E=1024, n_q=16, n_kv=8, D=128, n_rot=128, theta=1e6, FF=3072,
                           qtype=8, vocab=151936, eps=1e-6, positions="uniform32768"),
    "c3_qwen35_4b_prefill_bf16": dict(dtype="bf16", T=16384, E=2560, n_q=16, n_kv=4, D=256, n_rot=64, theta=1e7,
                                      FF=9216, qtype=2, vocab=248320, eps=1e-6, positions="range"),
    "c4_moe_bf16": dict(dtype="bf16", T=65536, E=2048, n_expert=256, n_used=8, FE=512, eps=1e-6),
    "c5_dense27b_bf16": dict(dtype="bf16", T=262144, E=5120, n_q=40, n_kv=8, D=128, n_rot=128, theta=1e6, FF=17408,
                             qtype=8, vocab=151936, eps=1e-6, positions="range"),
}
