"""The N > 1 path on CPU: two gloo ranks shard the rows as bench.py does, each runs its shard (here through the CPU
oracle, since no GPU is present), and the gathered result equals the unsharded one bit for bit; the max-over-ranks
reduction the benchmark uses for its device-timed duration is exercised on the same process group."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rocm_hip_b200.sharding import shard, shard_positions


def test_shard_ranges():
    for T in (1, 7, 64, 2427, 262144):
        for world in (1, 2, 3, 4, 8):
            rs = [shard(T, r, world) for r in range(world)]
            assert rs[0][0] == 0 and rs[-1][1] == T
            assert all(a[1] == b[0] for a, b in zip(rs, rs[1:]))
            sizes = [hi - lo for lo, hi in rs]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    from rocm_hip_b200 import synth
    T, E, nq, nkv, D, pos0 = 101, 256, 4, 2, 64, 5000
    lo, hi = shard(T, rank, world)
    n = hi - lo
    # a rank regenerates only its own rows (counter-based generator)
    x = synth.normal(0, "sh.x", lo * E, n * E).reshape(n, E)
    a = synth.normal(0, "sh.a", lo * E, n * E).reshape(n, E)
    w = synth.normal(0, "sh.w", 0, E, 1.0, 0.1)
    xo, y = O.add_rmsnorm(x, a, w, 1e-6)
    q = synth.normal(0, "sh.q", lo * nq * D, n * nq * D).reshape(n, nq * D)
    k = synth.normal(0, "sh.k", lo * nkv * D, n * nkv * D).reshape(n, nkv * D)
    qo, ko = O.qk_norm_rope(q, k, None, None, nq, nkv, D, D, 0, None, shard_positions(pos0, lo), 1e6, 1e-6)
    parts = [None] * world
    dist.all_gather_object(parts, (lo, hi, y, xo, qo, ko))
    # the benchmark's timing reduction: max over ranks
    t = torch.tensor([10.0 + rank, 1.0 - rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.tolist() == [10.0 + world - 1, 1.0]
    dist.barrier()
    if rank == 0:
        parts.sort(key=lambda p: p[0])
        np.savez(os.path.join(out_dir, "gathered.npz"), y=np.concatenate([p[2] for p in parts]),
                 xo=np.concatenate([p[3] for p in parts]), qo=np.concatenate([p[4] for p in parts]),
                 ko=np.concatenate([p[5] for p in parts]))
    dist.destroy_process_group()


def test_two_ranks_equal_one(tmp_path, oracle):
    from rocm_hip_b200 import synth
    world, port = 2, _free_port()
    mp.start_processes(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    g = np.load(tmp_path / "gathered.npz")
    T, E, nq, nkv, D, pos0 = 101, 256, 4, 2, 64, 5000
    x = synth.normal(0, "sh.x", 0, T * E).reshape(T, E)
    a = synth.normal(0, "sh.a", 0, T * E).reshape(T, E)
    w = synth.normal(0, "sh.w", 0, E, 1.0, 0.1)
    xo, y = oracle.add_rmsnorm(x, a, w, 1e-6)
    q = synth.normal(0, "sh.q", 0, T * nq * D).reshape(T, nq * D)
    k = synth.normal(0, "sh.k", 0, T * nkv * D).reshape(T, nkv * D)
    qo, ko = oracle.qk_norm_rope(q, k, None, None, nq, nkv, D, D, 0, None, pos0, 1e6, 1e-6)
    for name, want in (("y", y), ("xo", xo), ("qo", qo), ("ko", ko)):
        assert np.array_equal(g[name].view(np.uint32), want.view(np.uint32)), name
