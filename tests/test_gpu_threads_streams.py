"""Launchers called from several host threads at once, each on its own stream (the reference's rule: initialise once,
then launch from any thread that owns its stream, src/gpu_ops.cpp:9-17): every thread gets the results a single
thread gets. ctypes drops the interpreter lock during a call, so the launchers really run concurrently."""
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_concurrent_threads_on_their_own_streams(ops):
    T, n, nq, nkv, D, E_, U = 257, 2048, 8, 2, 128, 64, 4
    g = torch.Generator(device="cuda").manual_seed(5)
    R = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x, a, w = R(T, n), R(T, n), 1 + 0.1 * R(n)
    q, k, qn, kn = R(T, nq * D), R(T, nkv * D), 1 + 0.1 * R(D), 1 + 0.1 * R(D)
    ids = torch.randint(0, E_, (9000, U), device="cuda", dtype=torch.int32, generator=g)    # a long batch: segment kernels
    torch.cuda.synchronize()                                # the side streams below do not wait for the default stream

    def work(stream, base):
        out = {}
        with torch.cuda.stream(stream):
            for rep in range(20):
                xo, y, act = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
                ops.gpu_add_rmsnorm(x, a, xo, w, y, n, T, 1e-6)
                ops.gpu_swiglu(x, a, act, T * n)
                qo, ko = torch.empty_like(q), torch.empty_like(k)
                ops.gpu_qk_norm_rope(q, k, qn, kn, qo, ko, nq, nkv, D, D, 0, None, base, T, 1e6 if base % 2 else 1e4, 1e-6)
                m = ids.numel()
                tok, pair = (torch.empty(m, dtype=torch.int32, device="cuda") for _ in range(2))
                mt = ops.gpu_moe_max_tiles(ids.shape[0], U, E_, 64)
                ntl, te, ts, tn = (torch.zeros(kk, dtype=torch.int32, device="cuda") for kk in (1, mt, mt, mt))
                ops.gpu_moe_group(ids, ids.shape[0], U, E_, 64, tok, pair, ntl, te, ts, tn,
                                  scratch=torch.empty(ops.gpu_moe_group_scratch_ints(ids.shape[0], U, E_), dtype=torch.int32, device="cuda"))
                out = dict(y=y, act=act, qo=qo, ko=ko, pair=pair)
            stream.synchronize()
        return out

    want = {b: work(torch.cuda.Stream(), b) for b in (0, 1, 2, 3)}
    got = {}

    def run(b):
        got[b] = work(torch.cuda.Stream(), b)
    threads = [threading.Thread(target=run, args=(b,)) for b in (0, 1, 2, 3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    for b in (0, 1, 2, 3):
        for key in want[b]:
            assert torch.equal(want[b][key], got[b][key]), (b, key)


def test_moe_group_work_memory_slots_with_three_callers(ops):
    """gpu_moe_group without a scratch argument takes its work memory from four slots inside the library, used in
    turn: up to four long groupings may be in flight on a device at once. Three threads, each on its own stream and
    each waiting for its call before the next, stay inside that limit and must all get the single-thread result."""
    E_, U, rows = 64, 4, 9000
    g = torch.Generator(device="cuda").manual_seed(6)
    ids = [torch.randint(0, E_, (rows, U), device="cuda", dtype=torch.int32, generator=g) for _ in range(3)]
    torch.cuda.synchronize()

    def group(i, stream):
        res = None
        with torch.cuda.stream(stream):
            for _ in range(10):
                m = ids[i].numel()
                tok, pair = (torch.empty(m, dtype=torch.int32, device="cuda") for _ in range(2))
                mt = ops.gpu_moe_max_tiles(rows, U, E_, 64)
                ntl, te, ts, tn = (torch.zeros(kk, dtype=torch.int32, device="cuda") for kk in (1, mt, mt, mt))
                ops.gpu_moe_group(ids[i], rows, U, E_, 64, tok, pair, ntl, te, ts, tn)      # the library's own slots
                stream.synchronize()
                res = (tok, pair, ntl, te, ts, tn)
        return res

    want = [group(i, torch.cuda.Stream()) for i in range(3)]
    got = [None] * 3

    def run(i):
        got[i] = group(i, torch.cuda.Stream())
    threads = [threading.Thread(target=run, args=(i,)) for i in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for i in range(3):
        n_tiles = int(want[i][2].item())
        assert int(got[i][2].item()) == n_tiles
        assert torch.equal(want[i][0], got[i][0]) and torch.equal(want[i][1], got[i][1])
        for k in (3, 4, 5):
            assert torch.equal(want[i][k][:n_tiles], got[i][k][:n_tiles])
