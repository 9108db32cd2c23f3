"""The chunk schedule of the host-buffer calls (b200_host_chunk_plan; host logic, no device): every row is covered
once, no chunk exceeds a slot, the first and the last chunks are small, the ramp is symmetric, and the number of
chunks (each costs fixed copy and launch overheads) stays low."""
import ctypes as C

import pytest

from rocm_hip_b200 import _lib


def plan(T, slot_rows, n_slots):
    buf = (C.c_longlong * 4096)()
    n = _lib.load().b200_host_chunk_plan(T, slot_rows, n_slots, buf, 4096)
    assert 0 <= n <= 4096
    return list(buf[:n])


@pytest.mark.parametrize("T,slot_rows,n_slots", [(16384, 1272, 4), (16384, 159, 6), (1, 1000, 4), (63, 1000, 4), (64, 1000, 4),
                                                  (1000, 37, 3), (262144, 1272, 4), (5000, 5000, 2), (5001, 5000, 2),
                                                  (300, 100000, 4), (12345, 640, 5), (7, 1, 2)])
def test_every_row_once_and_no_chunk_larger_than_a_slot(T, slot_rows, n_slots):
    p = plan(T, slot_rows, n_slots)
    assert sum(p) == T and all(0 < c <= slot_rows for c in p)
    assert len(p) <= T // max(1, min(slot_rows, 64)) + 2 * 16 + 2 * n_slots + 2


def test_ramp_shape_for_a_long_batch():
    p = plan(16384, 1272, 4)
    assert p[0] == 79 and p[-1] == 79                       # 1/16 of a slot first and last
    k = 0
    while p[k + 1] == 2 * p[k]:
        k += 1
    assert k >= 3 and p[:k + 1] == p[::-1][:k + 1]          # doubling up, halving down, the same steps
    assert max(p) == 1272 and len(p) <= 24


def test_small_slots_keep_equal_chunks():
    p = plan(16384, 159, 6)
    assert p[0] == 64 and p[1] == 128 and set(p[2:-3]) == {159} and p[-2:] == [128, 64]


def test_nothing_to_do():
    assert plan(0, 100, 4) == [] and plan(10, 0, 4) == [] and plan(10, 100, 0) == []
