"""gpu_embed_rows_static_scratch: the embedding gather for callers that may not allocate device memory (engines that
gave away all of HBM at start-up, serving loops that ban cudaMalloc). It keeps its id buffer and bad-id flag in an
array inside the library, so this test drives it straight through the C ABI with nothing but inputs and outputs, and
checks it bit for bit against the CPU oracle's gather and against the ordinary entry point that takes caller-owned
scratch. Two calls in a row, the second shorter and with other ids, prove that what the first call left in the shared
array does not leak into the second; one call uses the array to its last id.
Collected last on purpose (file name), so a run that stops at the first failure has already covered everything else."""
import ctypes as C

import numpy as np
import pytest
import torch

from rocm_hip_b200 import _lib, synth

pytestmark = pytest.mark.gpu
MAX_IDS = 262144


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_matches_oracle_and_scratch_taking_entry_point_twice_in_a_row(ops, oracle):
    lib = _lib.load()
    vocab, E = 5000, 1024
    table_h = synth.q8_0_table(11, "zz.tab", vocab, E)
    table = torch.from_numpy(table_h).cuda()
    row_bytes = table.shape[1]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, T in enumerate((4099, 257)):
        ids = synth.randint(11, f"zz.ids{call}", 0, T, 0, vocab).astype(np.int32)
        want = torch.full((T, E), float("nan"), device="cuda")
        scratch = torch.zeros(T, dtype=torch.int32, device="cuda")
        flag = torch.full((1,), 2**31 - 1, dtype=torch.int32, device="cuda")
        assert lib.gpu_embed_rows_host_ids(8, _p(table), row_bytes, vocab, C.c_void_p(ids.ctypes.data), _p(scratch),
                                           _p(want), E, T, 1.0, _p(flag), stream) == 0
        got = torch.full((T, E), float("nan"), device="cuda")
        before = ops.launch_count()
        assert lib.gpu_embed_rows_static_scratch(8, _p(table), row_bytes, vocab, C.c_void_p(ids.ctypes.data), _p(got), E,
                                                 T, 1.0, stream) == 0
        assert ops.launch_count() == before + 1      # one kernel per accepted call, counted like every launcher's
        torch.cuda.synchronize()
        st, cpu = oracle.embed_rows(oracle.Q8_0, table_h, row_bytes, vocab, ids, E)
        assert st == 0 and np.array_equal(got.cpu().numpy().view(np.uint32), cpu.view(np.uint32)), f"call {call}"
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), f"call {call}"
    # Q4_0 through the same array, with an embedding scale
    table4 = torch.from_numpy(synth.q4_0_table(11, "zz.tab4", vocab, E)).cuda()
    T = 1000
    ids = synth.randint(11, "zz.ids4", 0, T, 0, vocab).astype(np.int32)
    want, got = torch.zeros(T, E, device="cuda"), torch.zeros(T, E, device="cuda")
    scratch = torch.zeros(T, dtype=torch.int32, device="cuda")
    flag = torch.full((1,), 2**31 - 1, dtype=torch.int32, device="cuda")
    assert lib.gpu_embed_rows_host_ids(2, _p(table4), table4.shape[1], vocab, C.c_void_p(ids.ctypes.data), _p(scratch),
                                       _p(want), E, T, 0.5, _p(flag), stream) == 0
    assert lib.gpu_embed_rows_static_scratch(2, _p(table4), table4.shape[1], vocab, C.c_void_p(ids.ctypes.data), _p(got),
                                             E, T, 0.5, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))


def test_a_call_at_exactly_the_ceiling(ops, oracle):
    """T = 262,144 ids fill the built-in array to its last entry (the flag word sits right behind it)."""
    lib = _lib.load()
    vocab, E, T = 64, 32, MAX_IDS
    table_h = synth.q8_0_table(13, "zz.ceil", vocab, E)
    table = torch.from_numpy(table_h).cuda()
    ids = synth.randint(13, "zz.ceil.ids", 0, T, 0, vocab).astype(np.int32)
    ids[-1] = vocab - 1
    got = torch.full((T, E), float("nan"), device="cuda")
    assert lib.gpu_embed_rows_static_scratch(8, _p(table), table.shape[1], vocab, C.c_void_p(ids.ctypes.data), _p(got), E,
                                             T, 1.0, None) == 0
    torch.cuda.synchronize()
    st, cpu = oracle.embed_rows(oracle.Q8_0, table_h, table.shape[1], vocab, ids, E)
    assert st == 0 and np.array_equal(got.cpu().numpy().view(np.uint32), cpu.view(np.uint32))


def test_limits_are_refused_without_queueing_anything(ops):
    lib = _lib.load()
    vocab, E = 64, 32
    table = torch.from_numpy(synth.q8_0_table(12, "zz.small", vocab, E)).cuda()
    out = torch.zeros(8, E, device="cuda")
    before = ops.launch_count()
    too_many = np.zeros(MAX_IDS + 1, dtype=np.int32)
    assert lib.gpu_embed_rows_static_scratch(8, _p(table), table.shape[1], vocab, C.c_void_p(too_many.ctypes.data), _p(out),
                                             E, MAX_IDS + 1, 1.0, None) == _lib.cudaErrorInvalidValue
    bad = np.array([1, 2, vocab, 3], dtype=np.int32)
    assert lib.gpu_embed_rows_static_scratch(8, _p(table), table.shape[1], vocab, C.c_void_p(bad.ctypes.data), _p(out), E,
                                             4, 1.0, None) == _lib.cudaErrorInvalidValue
    # only Q8_0 (8) and Q4_0 (2) tables: another row format is refused, not misread
    ok = np.array([1, 2, 3, 4], dtype=np.int32)
    f16 = torch.zeros(vocab, E, dtype=torch.float16, device="cuda")
    assert lib.gpu_embed_rows_static_scratch(1, _p(f16), 2 * E, vocab, C.c_void_p(ok.ctypes.data), _p(out), E, 4, 1.0,
                                             None) == _lib.cudaErrorInvalidValue
    torch.cuda.synchronize()
    assert not out.any() and ops.launch_count() == before
    # before gpu_ops_init the entry point answers like every launcher
    ops.gpu_ops_free()
    try:
        assert lib.gpu_embed_rows_static_scratch(8, _p(table), table.shape[1], vocab, C.c_void_p(ok.ctypes.data), _p(out),
                                                 E, 4, 1.0, None) == _lib.cudaErrorInvalidDeviceFunction
    finally:
        assert ops.gpu_ops_init("gpu_ops.co") == 0
