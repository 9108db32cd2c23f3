"""CUDA embedding gather + dequantisation against the CPU oracle through the C ABI: bit-exact (memcmp), as the
reference's dequant_verify demands of its decoders (tests/dequant_verify.cpp:106-125)."""
import os

import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import dev, host

pytestmark = pytest.mark.gpu
INT_MAX = 2**31 - 1


def gather(ops, qt, table, vocab, ids, E, scale=1.0, bf16=False, row_bytes=None):
    T = ids.size
    dt = dev(table)
    out = torch.full((T, E), float("nan"), device="cuda", dtype=torch.bfloat16 if bf16 else torch.float32)
    bad = ops.gpu_embed_rows(qt, dt, row_bytes or table.shape[1], vocab, dev(ids.astype(np.int32)), out, E, T, scale)
    torch.cuda.synchronize()
    return host(out), int(bad.item())


def test_c1_q8_0_full_table(ops, oracle):
    """Qwen3-0.6B: Q8_0 table 151,936 x 1,024 (165 MB), 2,427 ids uniform over the vocabulary."""
    vocab, E, T = 151936, 1024, 2427
    table = synth.q8_0_table(0, "c1.embd", vocab, E)
    ids = synth.randint(0, "c1.ids", 0, T, 0, vocab)
    st, want = oracle.embed_rows(oracle.Q8_0, table, table.shape[1], vocab, ids, E)
    got, bad = gather(ops, ops.QT_Q8_0, table, vocab, ids, E)
    assert st == 0 and bad == INT_MAX
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    got, _ = gather(ops, ops.QT_Q8_0, table, vocab, ids, E, bf16=True)
    _, want = oracle.embed_rows(oracle.Q8_0, table, table.shape[1], vocab, ids, E, bf16=True)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("E", [32, 96, 256, 2560, 5120, 8192])
def test_q4_0_and_q8_0_widths(ops, oracle, E):
    """Row widths whose byte length is and is not a multiple of 16 (staging by 16-byte or 2-byte loads), rows longer
    than one staging chunk (8192), fp32 and bf16 outputs, every row of the table once plus repeats."""
    vocab = 777
    for qt, maker in ((oracle.Q8_0, synth.q8_0_table), (oracle.Q4_0, synth.q4_0_table)):
        table = maker(1, f"w{E}", vocab, E)
        ids = np.concatenate([np.arange(vocab), synth.randint(1, "w.ids", 0, 300, 0, vocab)])
        for bf16 in (False, True):
            st, want = oracle.embed_rows(qt, table, table.shape[1], vocab, ids, E, bf16=bf16)
            got, bad = gather(ops, qt, table, vocab, ids, E, bf16=bf16)
            assert st == 0 and bad == INT_MAX and np.array_equal(got.view(np.uint8), want.view(np.uint8))


def test_golden_tables(ops):
    """The reference's own decode of tables with special fp16 scales (zero, subnormal, largest), tests/golden/dequant.npz."""
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "dequant.npz"))
    for name, qt in (("q8_0", 8), ("q4_0", 2)):
        table, want = g[name + "_table"], g[name + "_out"]
        rows, E = want.shape
        got, bad = gather(ops, qt, table, rows, np.arange(rows), E)
        assert bad == INT_MAX and np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_embedding_scale_and_row_stride(ops, oracle):
    vocab, E = 100, 256
    table = synth.q8_0_table(2, "sc", vocab, E)
    ids = synth.randint(2, "sc.ids", 0, 64, 0, vocab)
    _, want = oracle.embed_rows(oracle.Q8_0, table, table.shape[1], vocab, ids, E, scale=16.0)
    got, _ = gather(ops, 8, table, vocab, ids, E, scale=16.0)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    _, want = oracle.embed_rows(oracle.Q8_0, table, table.shape[1], vocab, ids, E, scale=0.3)
    got, _ = gather(ops, 8, table, vocab, ids, E, scale=0.3)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # rows at a stride larger than their payload
    stride = table.shape[1] + 6
    padded = np.zeros((vocab, stride), dtype=np.uint8)
    padded[:, : table.shape[1]] = table
    _, want = oracle.embed_rows(oracle.Q8_0, padded, stride, vocab, ids, E)
    got, _ = gather(ops, 8, padded, vocab, ids, E, row_bytes=stride)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_out_of_range_ids(ops, oracle):
    """An id outside [0, vocab) (src/qwen_model.cpp:981) is reported through the flag as the first offending row,
    its row is zero-filled, the table is not read there, and the other rows are still right. The host-id entry point
    refuses before launching anything."""
    vocab, E, T = 50, 128, 40
    table = synth.q8_0_table(3, "bad", vocab, E)
    ids = synth.randint(3, "bad.ids", 0, T, 0, vocab).astype(np.int32)
    good = ids.copy()
    ids[[7, 23]] = [vocab, -5]
    got, bad = gather(ops, 8, table, vocab, ids, E)
    assert bad == 7
    assert not got[7].any() and not got[23].any()
    _, want = oracle.embed_rows(oracle.Q8_0, table, table.shape[1], vocab, good, E)
    keep = np.ones(T, bool); keep[[7, 23]] = False
    assert np.array_equal(got[keep].view(np.uint32), want[keep].view(np.uint32))
    assert oracle.embed_rows(oracle.Q8_0, table, table.shape[1], vocab, ids, E)[0] == -1

    import ctypes as C
    from rocm_hip_b200 import _lib
    lib = _lib.load()
    out = torch.zeros(T, E, device="cuda")
    scratch = torch.zeros(T, dtype=torch.int32, device="cuda")
    flag = torch.full((1,), INT_MAX, dtype=torch.int32, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    before = ops.launch_count()
    code = lib.gpu_embed_rows_host_ids(8, p(dev(table)), table.shape[1], vocab, C.c_void_p(ids.ctypes.data), p(scratch),
                                       p(out), E, T, 1.0, p(flag), None)
    assert code == 1 and ops.launch_count() == before
    dt = dev(table)
    code = lib.gpu_embed_rows_host_ids(8, p(dt), table.shape[1], vocab, C.c_void_p(good.ctypes.data), p(scratch),
                                       p(out), E, T, 1.0, p(flag), None)
    torch.cuda.synchronize()
    assert code == 0 and np.array_equal(host(out).view(np.uint32), want.view(np.uint32))


def test_argument_errors(ops):
    t = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    ids = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.zeros(4, 64, device="cuda")
    for qt, E, rb in ((9, 64, 68), (8, 48, 68), (8, 64, 60), (8, 64, 69)):
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_embed_rows(qt, t, rb, 10, ids, out, E, 4)
        assert e.value.code == 1


ALL_FORMATS = ["QT_F32", "QT_F16", "QT_BF16", "QT_Q4_1", "QT_Q5_0", "QT_Q5_1", "QT_Q4_K", "QT_Q5_K", "QT_Q6_K"]


@pytest.mark.parametrize("fmt", ALL_FORMATS)
@pytest.mark.parametrize("E", [512, 5120, 2304])
def test_other_row_formats_bit_exact(ops, oracle, fmt, E):
    """The other formats a token_embd.weight comes in (src/quant_types.cpp:58-74,126-179,264-345): fp32 and bf16 output,
    with and without an embedding scale, a row stride larger than the row, bad ids -- bit for bit against the oracle,
    whose decoders are pinned to the reference build's qt_to_float."""
    qt = getattr(ops, fmt)
    vocab, T = 300, 517
    table = synth.gguf_table(5, "emb." + fmt, qt, vocab, E)
    assert ops.qt_row_size(qt, E) == table.shape[1]
    ids = synth.randint(5, "emb.ids", 0, T, 0, vocab).astype(np.int32)
    dt, d_ids = dev(table), dev(ids)
    for scale in (1.0, 0.0625 * 3):
        out = torch.zeros(T, E, device="cuda")
        flag = ops.gpu_embed_rows(qt, dt, table.shape[1], vocab, d_ids, out, E, T, scale)
        torch.cuda.synchronize()
        st, want = oracle.embed_rows(qt, table, table.shape[1], vocab, ids, E, scale)
        assert st == 0 and int(flag.item()) == 2**31 - 1
        assert np.array_equal(host(out).view(np.uint32), want.view(np.uint32))
        ob = torch.zeros(T, E, device="cuda", dtype=torch.bfloat16)
        ops.gpu_embed_rows(qt, dt, table.shape[1], vocab, d_ids, ob, E, T, scale)
        torch.cuda.synchronize()
        _, wb = oracle.embed_rows(qt, table, table.shape[1], vocab, ids, E, scale, bf16=True)
        assert np.array_equal(host(ob), wb)
    # rows at a stride (2 extra bytes: rows no longer 16-byte aligned -> the 2-byte staging path), and a bad id
    wide = np.zeros((vocab, table.shape[1] + 2), np.uint8)
    wide[:, :table.shape[1]] = table
    bad = ids.copy()
    bad[77] = vocab + 5
    out = torch.full((T, E), -1.0, device="cuda")
    flag = ops.gpu_embed_rows(qt, dev(wide), wide.shape[1], vocab, dev(bad), out, E, T, 1.0)
    torch.cuda.synchronize()
    _, want = oracle.embed_rows(qt, table, table.shape[1], vocab, ids, E)
    got = host(out)
    assert int(flag.item()) == 77 and not got[77].any()
    keep = np.arange(T) != 77
    assert np.array_equal(got[keep].view(np.uint32), want[keep].view(np.uint32))


@pytest.mark.parametrize("fmt", ALL_FORMATS)
@pytest.mark.parametrize("E", [5120, 2304, 256])
def test_other_row_formats_long_batches(ops, oracle, fmt, E):
    """Long batches of the other formats (a slice-per-warp kernel for them measured faster only for Q4_K, 0.75 against
    0.71 of the copy bandwidth, and slower for Q5_1 and Q6_K, so they keep the whole-row kernel): the same bits, bad ids
    as zero rows and the first bad index."""
    qt = getattr(ops, fmt)
    vocab, T = 200, 9001
    table = synth.gguf_table(6, "embl." + fmt, qt, vocab, E)
    ids = synth.randint(6, "embl.ids", 0, T, 0, vocab).astype(np.int32)
    ids[[4000, 8999]] = [vocab, -3]
    good = ids.copy()
    good[[4000, 8999]] = 0
    dt, d_ids = dev(table), dev(ids)
    out = torch.full((T, E), -1.0, device="cuda")
    flag = ops.gpu_embed_rows(qt, dt, table.shape[1], vocab, d_ids, out, E, T, 1.0)
    ob = torch.zeros(T, E, device="cuda", dtype=torch.bfloat16)
    ops.gpu_embed_rows(qt, dt, table.shape[1], vocab, d_ids, ob, E, T, 0.1875)
    torch.cuda.synchronize()
    _, want = oracle.embed_rows(qt, table, table.shape[1], vocab, good, E)
    _, wb = oracle.embed_rows(qt, table, table.shape[1], vocab, good, E, 0.1875, bf16=True)
    got, gb = host(out), host(ob)
    assert int(flag.item()) == 4000 and not got[4000].any() and not got[8999].any() and not gb[4000].any()
    keep = np.ones(T, bool)
    keep[[4000, 8999]] = False
    assert np.array_equal(got[keep].view(np.uint32), want[keep].view(np.uint32))
    assert np.array_equal(gb[keep], wb[keep])


def test_k_formats_need_whole_super_blocks(ops):
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    ids = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.zeros(4, 128, device="cuda")
    with pytest.raises(ops.LayerOpError) as e:
        ops.gpu_embed_rows(ops.QT_Q6_K, t, 210, 16, ids, out, 128, 4, 1.0)      # 128 is not a multiple of 256
    assert e.value.code == 1
    with pytest.raises(ops.LayerOpError):
        ops.gpu_embed_rows(9, t, 64, 16, ids, out, 128, 4, 1.0)                 # ggml id 9 (Q8_1) is not a row format


@pytest.mark.parametrize("qt,E", [(8, 2048), (2, 2560), (8, 256)])
@pytest.mark.parametrize("T", [60, 50000])
def test_every_batch_length_gives_the_oracle_rows(ops, oracle, qt, E, T):
    """The launcher picks its kernel from the batch length and the row shape (a few tokens per resident warp: slices
    of a row in flight as bulk copies; long batches: a warp per slice, one slice per warp; other shapes: whole-row
    load -> decode). Whatever runs, every row is the oracle's to the bit, in fp32 and rounded once to bf16, and ids
    out of range give zero rows and the first offending row index."""
    vocab = 300
    maker, okind = (synth.q8_0_table, oracle.Q8_0) if qt == 8 else (synth.q4_0_table, oracle.Q4_0)
    table = maker(21, "len.tab", vocab, E)
    ids = synth.randint(21, "len.ids", 0, T, 0, vocab).astype(np.int32)
    _, want = oracle.embed_rows(okind, table, table.shape[1], vocab, ids, E)
    got, bad = gather(ops, qt, table, vocab, ids, E)
    assert bad == INT_MAX and np.array_equal(got.view(np.uint32), want.view(np.uint32))
    got16, bad = gather(ops, qt, table, vocab, ids, E, bf16=True)
    assert bad == INT_MAX and np.array_equal(got16, oracle.f32_to_bf16(want).reshape(T, E))
    ids2 = ids.copy()
    ids2[[T // 3, T - 2]] = [vocab + 7, -1]
    got, bad = gather(ops, qt, table, vocab, ids2, E)
    assert bad == T // 3 and not got[T // 3].any() and not got[T - 2].any()
    keep = np.ones(T, bool)
    keep[[T // 3, T - 2]] = False
    assert np.array_equal(got[keep].view(np.uint32), want[keep].view(np.uint32))
