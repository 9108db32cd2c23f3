"""gpu_moe_group against a numpy statement of the reference's contract (src/gpu_ops.hip:259-320): entries sorted by
expert, runs cut into tiles, counts and tiles exact; here also the order inside a run (ascending pair index). Then
the expert-grouped SwiGLU rows of the MoE configuration built from it."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import bf16_ulp_dist, dev, host

pytestmark = pytest.mark.gpu


def reference_grouping(ids, n_expert, tile):
    flat = ids.ravel()
    order = np.argsort(flat, kind="stable")          # by expert, ties by pair index
    counts = np.bincount(flat, minlength=n_expert)
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    te, ts, tn = [], [], []
    for e in range(n_expert):
        for k in range(0, counts[e], tile):
            te.append(e); ts.append(starts[e] + k); tn.append(min(tile, counts[e] - k))
    return order, np.array(te), np.array(ts), np.array(tn)


@pytest.mark.parametrize("T,n_used,n_expert,tile", [(8, 8, 256, 16), (2048, 8, 256, 64), (333, 4, 60, 32), (1, 8, 128, 16),
                                                      (5000, 8, 256, 128), (700, 2, 1024, 8)])
def test_grouping(ops, T, n_used, n_expert, tile):
    ids, _ = synth.moe_routing(T, "mg.route", T, n_expert, n_used)
    d_ids = dev(ids)
    n = T * n_used
    mt = ops.gpu_moe_max_tiles(T, n_used, n_expert, tile)
    z = lambda k: torch.full((k,), -7, dtype=torch.int32, device="cuda")
    tok, pair, ntl, te, ts, tn = z(n), z(n), z(1), z(mt + 4), z(mt + 4), z(mt + 4)
    for _ in range(2):    # twice: the result is deterministic
        ops.gpu_moe_group(d_ids, T, n_used, n_expert, tile, tok, pair, ntl, te, ts, tn)
        torch.cuda.synchronize()
        order, wte, wts, wtn = reference_grouping(ids, n_expert, tile)
        k = int(ntl.item())
        assert k == len(wte) <= mt
        assert np.array_equal(host(te)[:k], wte) and np.array_equal(host(ts)[:k], wts) and np.array_equal(host(tn)[:k], wtn)
        assert (host(te)[mt:] == -7).all()
        assert np.array_equal(host(pair), order) and np.array_equal(host(tok), order // n_used)


@pytest.mark.parametrize("T,n_used,n_expert,tile", [(1025, 8, 256, 64), (20000, 8, 128, 64), (65536, 8, 256, 128),
                                                      (4099, 3, 1000, 16), (300000, 4, 60, 256), (9000, 1, 7, 32)])
def test_long_batches_take_the_segment_kernels(ops, T, n_used, n_expert, tile):
    """More than 8192 entries: three launches over the whole device, the same arrays as the one-CTA kernel would write
    (the numpy statement), deterministic, with the library's scratch slots and with the caller's."""
    ids, _ = synth.moe_routing(T, "mg.long", T, n_expert, n_used)
    ids = ids.copy()
    ids.ravel()[5::997] = -1                      # entries to skip, as the one-CTA kernel skips them
    ids.ravel()[7::1013] = n_expert
    d_ids = dev(ids)
    n = T * n_used
    assert n > 8192
    flat = ids.ravel()
    keep = np.flatnonzero((flat >= 0) & (flat < n_expert))
    order = keep[np.argsort(flat[keep], kind="stable")]
    counts = np.bincount(flat[keep], minlength=n_expert)
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    wte = np.concatenate([np.full((c + tile - 1) // tile, e) for e, c in enumerate(counts)])
    wts = np.concatenate([starts[e] + tile * np.arange((c + tile - 1) // tile) for e, c in enumerate(counts)])
    wtn = np.concatenate([np.minimum(tile, c - tile * np.arange((c + tile - 1) // tile)) for e, c in enumerate(counts)])
    mt = ops.gpu_moe_max_tiles(T, n_used, n_expert, tile)
    z = lambda k: torch.full((k,), -7, dtype=torch.int32, device="cuda")
    need = ops.gpu_moe_group_scratch_ints(T, n_used, n_expert)
    assert 0 < need <= 1024 * n_expert
    for scratch in (None, None, None, None, None, z(need)):     # the library's slots in turn, then the caller's
        tok, pair, ntl, te, ts, tn = z(n), z(n), z(1), z(mt + 4), z(mt + 4), z(mt + 4)
        before = ops.launch_count()
        ops.gpu_moe_group(d_ids, T, n_used, n_expert, tile, tok, pair, ntl, te, ts, tn, scratch=scratch)
        torch.cuda.synchronize()
        assert ops.launch_count() - before == 3
        k = int(ntl.item())
        assert k == len(wte) <= mt
        assert np.array_equal(host(te)[:k], wte) and np.array_equal(host(ts)[:k], wts) and np.array_equal(host(tn)[:k], wtn)
        assert (host(te)[mt:] == -7).all()
        m = len(order)
        assert np.array_equal(host(pair)[:m], order) and np.array_equal(host(tok)[:m], order // n_used)
        assert (host(pair)[m:] == -7).all()
    with pytest.raises(ops.LayerOpError):
        ops.gpu_moe_group(d_ids, T, n_used, n_expert, tile, tok, pair, ntl, te, ts, tn, scratch=z(need - 1))
    assert ops.gpu_moe_group_scratch_ints(1024, 8, 256) == 0


def test_argument_errors(ops):
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    o = torch.zeros(64, dtype=torch.int32, device="cuda")
    for T, nu, ne, tile in ((0, 8, 256, 16), (1, 0, 256, 16), (1, 8, 0, 16), (1, 8, 1025, 16), (1, 8, 256, 0)):
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_moe_group(ids, T, nu, ne, tile, o, o, o, o, o, o)
        assert e.value.code == 1


def test_expert_grouped_swiglu_rows(ops, oracle):
    """MoE shape at a reduced token count: top-8 of 256 experts, expert width 512; the gate / up rows are gathered in
    the order gpu_moe_group produced, and SwiGLU over the grouped rows equals the oracle on the same rows."""
    T, n_used, n_expert, FE = 512, 8, 256, 512
    ids, _ = synth.moe_routing(0, "mg.c4", T, n_expert, n_used)
    n = T * n_used
    tok, pair = (torch.zeros(n, dtype=torch.int32, device="cuda") for _ in range(2))
    mt = ops.gpu_moe_max_tiles(T, n_used, n_expert, 64)
    ntl, te, ts, tn = (torch.zeros(k, dtype=torch.int32, device="cuda") for k in (1, mt, mt, mt))
    ops.gpu_moe_group(dev(ids), T, n_used, n_expert, 64, tok, pair, ntl, te, ts, tn)
    g = oracle.f32_to_bf16(synth.normal(0, "mg.g", 0, n * FE)).reshape(n, FE)
    u = oracle.f32_to_bf16(synth.normal(0, "mg.u", 0, n * FE)).reshape(n, FE)
    idx = pair.long()
    gg = dev(g, torch.bfloat16)[idx].contiguous()
    uu = dev(u, torch.bfloat16)[idx].contiguous()
    out = torch.zeros_like(gg)
    ops.gpu_swiglu(gg, uu, out, n * FE)
    torch.cuda.synchronize()
    p = host(pair)
    assert bf16_ulp_dist(host(out), oracle.swiglu_bf16(g[p], u[p]).reshape(n, FE)).max() <= 1
    experts = ids.ravel()[p]
    assert (np.diff(experts) >= 0).all()       # rows are grouped by expert id
