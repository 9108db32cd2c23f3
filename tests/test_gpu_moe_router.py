"""The MoE routers behind their reference-named launchers (src/gpu_ops.h:30-37, 119-124): expert selection exact
(descending, ties to the lower index), weights and the shared-expert gate to 1e-6 against the oracle's statement of
the kernels (src/gpu_ops.hip:150-241, 794-824); relu2; and router -> group -> combine as one chain."""
import numpy as np
import pytest
import torch

from rocm_hip_b200 import synth
from util import dev, host

pytestmark = pytest.mark.gpu


def _logits(T, n_expert, seed, ties=True):
    l = synth.normal(seed, "rt.l", 0, T * n_expert).reshape(T, n_expert) * 2
    if ties and n_expert >= 8:
        l[0, :] = 0.5                                  # all equal: experts 0 .. n_used - 1 in order
        l[1, 3] = l[1, n_expert - 1] = l[1].max() + 1  # a tie for first place: the lower index first
        l[2, ::2] = l[2, 1::2][: l[2, ::2].size]       # many pairs of equal values
    return l


@pytest.mark.parametrize("T,n_expert,n_used,n,stride", [(300, 256, 8, 2048, 0), (77, 60, 4, 1000, 6), (33, 128, 8, 5120, 9),
                                                          (9, 1024, 64, 512, 0), (50, 512, 40, 777, 0), (5, 32, 32, 64, 33),
                                                          (4, 8, 1, 16, 0)])
def test_softmax_router(ops, oracle, T, n_expert, n_used, n, stride):
    l = _logits(T, n_expert, 1)
    x = synth.normal(1, "rt.x", 0, T * n).reshape(T, n)
    w = synth.normal(1, "rt.w", 0, n, 0.0, 0.05)
    st = stride or n_used
    for gate in (True, False):
        ids = torch.full((T, st), -5, dtype=torch.int32, device="cuda")
        wts = torch.zeros(T, n_used, device="cuda")
        sg = torch.full((T,), -5.0, device="cuda")
        ops.gpu_moe_router(dev(l), dev(x) if gate else None, dev(w) if gate else None, ids, wts, sg if gate else None,
                           n_expert, n_used, n, T, ids_stride=stride)
        torch.cuda.synchronize()
        wi, ww, wsg = oracle.moe_router(l, n_used, x if gate else None, w if gate else None)
        gi = host(ids)
        assert np.array_equal(gi[:, :n_used], wi)
        if st > n_used:
            assert (gi[:, n_used] == -1).all() and (gi[:, n_used + 1:] == -5).all()
        assert np.abs(host(wts) - ww).max() <= 1e-6 and np.allclose(host(wts).sum(axis=1), 1.0, atol=1e-5)
        assert (np.diff(host(wts), axis=1) <= 0).all()             # descending
        if gate:
            assert np.abs(host(sg) - wsg).max() <= 2e-6
        else:
            assert (host(sg) == -5.0).all()


@pytest.mark.parametrize("T,n_expert,n_used,norm,scale", [(200, 128, 6, 1, 2.5), (50, 512, 22, 0, 1.0), (31, 60, 4, 1, 1.0),
                                                            (8, 1024, 64, 0, 0.5)])
def test_sigmoid_router(ops, oracle, T, n_expert, n_used, norm, scale):
    l = _logits(T, n_expert, 2)
    bias = synth.normal(2, "rt.b", 0, n_expert, 0.0, 0.2)
    ids = torch.zeros(T, n_used, dtype=torch.int32, device="cuda")
    wts = torch.zeros(T, n_used, device="cuda")
    ops.gpu_moe_router_sigmoid(dev(l), dev(bias), ids, wts, n_expert, n_used, norm, scale, T)
    torch.cuda.synchronize()
    wi, ww = oracle.moe_router_sigmoid(l, bias, n_used, norm, scale)
    assert np.array_equal(host(ids), wi)
    assert np.abs(host(wts) - ww).max() <= 2e-6 * max(1.0, scale)


def test_router_argument_errors(ops):
    l = torch.zeros(4, 64, device="cuda")
    ids = torch.zeros(4, 8, dtype=torch.int32, device="cuda")
    w = torch.zeros(4, 8, device="cuda")
    for ne, nu, T, st in ((0, 8, 4, 0), (1025, 8, 4, 0), (64, 0, 4, 0), (64, 65, 4, 0), (16, 17, 4, 0), (64, 8, 0, 0),
                          (64, 8, 4, 7)):
        with pytest.raises(ops.LayerOpError) as e:
            ops.gpu_moe_router(l, None, None, ids, w, None, ne, nu, 0, T, ids_stride=st)
        assert e.value.code == 1


@pytest.mark.parametrize("rows,h,stride", [(40, 1024, 1024), (33, 500, 640), (7, 37, 41)])
def test_relu2(ops, oracle, rows, h, stride):
    buf = synth.normal(3, "r2.x", 0, rows * stride).reshape(rows, stride)
    out = torch.empty(rows, h, device="cuda")
    ops.gpu_relu2(dev(buf), out, rows, h, stride)
    torch.cuda.synchronize()
    assert np.array_equal(host(out).view(np.uint32), oracle.relu2(buf[:, :h]).view(np.uint32))
    if (rows * h) % 256 == 0:
        q8 = ops.Q8Buffers(rows * h, "cuda", xh="bf16")
        ops.gpu_relu2(dev(buf), out, rows, h, stride, q8=q8)
        torch.cuda.synchronize()
        want = oracle.quantize_q8(host(out), xh="bf16")
        for k in ("q0", "d0", "s0", "qK", "dK", "bsK"):
            assert np.array_equal(host(getattr(q8, k)).view(want[k].dtype), want[k]), k
    with pytest.raises(ops.LayerOpError):
        ops.gpu_relu2(dev(buf), out, rows, h, h - 1)


def test_router_group_combine_chain(ops, oracle):
    """The MoE bookkeeping of one layer on the device: route, group by expert, (the experts' matmuls stand-in: each
    pair's row is its expert's vector), combine -- against the same chain on the oracle."""
    T, n_expert, n_used, n = 700, 64, 4, 256
    l = _logits(T, n_expert, 4, ties=False)
    ids = torch.zeros(T, n_used, dtype=torch.int32, device="cuda")
    wts = torch.zeros(T, n_used, device="cuda")
    ops.gpu_moe_router(dev(l), None, None, ids, wts, None, n_expert, n_used, 0, T)
    m = T * n_used
    tok, pair = (torch.zeros(m, dtype=torch.int32, device="cuda") for _ in range(2))
    mt = ops.gpu_moe_max_tiles(T, n_used, n_expert, 32)
    ntl, te, ts, tn = (torch.zeros(k, dtype=torch.int32, device="cuda") for k in (1, mt, mt, mt))
    ops.gpu_moe_group(ids, T, n_used, n_expert, 32, tok, pair, ntl, te, ts, tn)
    expert_vec = synth.normal(4, "ch.e", 0, n_expert * n).reshape(n_expert, n)
    d_ev = dev(expert_vec)
    down = torch.zeros(m, n, device="cuda")
    k = int(ntl.item())
    for i in range(k):                                   # "expert e processes its tile": rows pair_rows[start : start + n]
        e, s, c = int(te[i]), int(ts[i]), int(tn[i])
        down[pair[s:s + c].long()] = d_ev[e]
    out = torch.empty(T, n, device="cuda")
    ops.gpu_moe_combine(down.view(T, n_used, n), wts, None, None, out, n_used, n, T)
    torch.cuda.synchronize()
    wi, ww, _ = oracle.moe_router(l, n_used)
    want = oracle.moe_combine(expert_vec[wi], ww)
    assert np.array_equal(host(ids), wi)
    assert np.abs(host(out) - want).max() <= 1e-5
