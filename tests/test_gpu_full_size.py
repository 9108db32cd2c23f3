"""The dense-27B configuration at its full row count (262,144 tokens, hidden 5120, 40 + 8 heads of 128, intermediate
17408, Q8_0 table 151,936 x 5120; bf16), where the CPU oracle would take minutes: each kernel is checked over EVERY
row through properties that do not depend on size, evaluated on the device with plain torch arithmetic in chunks
(an independent statement of the same math, not the kernels under test):
  * exact ones: the stored residual sum, the embedding decode, shard-by-shard == whole batch (bit for bit);
  * bounded ones: outputs within 2 bf16 ulp of a float32 / float64 torch evaluation, rotation keeps pair norms.
The small-size tests pin the bits against the reference; these pin the absence of size-dependent faults (64-bit
offsets, grid-stride tails, tile remainders)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
T, E, NQ, NKV, D, FF, VOCAB = 262144, 5120, 40, 8, 128, 17408, 151936
CH = 16384
bf = torch.bfloat16


def ulp_dist(a, b):
    """bf16 tensors -> int tensor of ulp distances."""
    def key(t):
        u = t.view(torch.int16).to(torch.int32) & 0xFFFF
        return torch.where(u >= 0x8000, -(u & 0x7FFF), u)
    return (key(a) - key(b)).abs()


def rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = torch.empty(shape, device="cuda", dtype=bf)
    for r in range(0, shape[0], CH):
        out[r:r + CH] = (torch.randn((min(CH, shape[0] - r),) + tuple(shape[1:]), device="cuda", generator=g) * scale).to(bf)
    return out


def test_add_rmsnorm_full(ops):
    x, a = rand((T, E), 1), rand((T, E), 2)
    w = 1 + 0.1 * torch.randn(E, device="cuda")
    xo, y = torch.empty_like(x), torch.empty_like(x)
    ops.gpu_add_rmsnorm(x, a, xo, w, y, E, T, 1e-6)
    y_plain = torch.empty_like(x)
    ops.gpu_add_rmsnorm(xo, None, xo, w, y_plain, E, T, 1e-6)       # unfused: norm of the stored sum
    assert torch.equal(y_plain.view(torch.int16), y.view(torch.int16))
    worst = 0
    for r in range(0, T, CH):
        s = (x[r:r + CH].float() + a[r:r + CH].float())
        assert torch.equal(xo[r:r + CH].view(torch.int16), s.to(bf).view(torch.int16))
        v = xo[r:r + CH].double()
        ref = (v * torch.rsqrt((v * v).mean(dim=1, keepdim=True) + 1e-6)).float() * w
        worst = max(worst, int(ulp_dist(y[r:r + CH], ref.to(bf)).max()))
    assert worst <= 1
    # two shards give the whole batch's bits
    h = T // 2 + 37
    y2 = torch.empty_like(x)
    ops.gpu_add_rmsnorm(x[:h], a[:h], xo[:h], w, y2[:h], E, h, 1e-6)
    ops.gpu_add_rmsnorm(x[h:], a[h:], xo[h:], w, y2[h:], E, T - h, 1e-6)
    assert torch.equal(y2.view(torch.int16), y.view(torch.int16))


def test_swiglu_full(ops):
    n = T * FF                                    # 4.56e9 values: beyond 32-bit indexing
    g, u = rand((T, FF), 3, 2.0), rand((T, FF), 4)
    out = torch.empty_like(g)
    ops.gpu_swiglu(g, u, out, n)
    worst, diff = 0, 0
    for r in range(0, T, CH):
        gf, uf = g[r:r + CH].float(), u[r:r + CH].float()
        ref = (gf / (1 + torch.exp(-gf)) * uf).to(bf)
        d = ulp_dist(out[r:r + CH], ref)
        worst = max(worst, int(d.max()))
        diff += int((d != 0).sum())
    assert worst <= 1 and diff < n * 1e-3
    assert torch.isfinite(out[-1].float()).all() and out[-1].float().abs().sum() > 0   # the last row was written


def test_qk_norm_rope_full(ops):
    q, k = rand((T, NQ * D), 5), rand((T, NKV * D), 6)
    qn = 1 + 0.1 * torch.randn(D, device="cuda")
    kn = 1 + 0.1 * torch.randn(D, device="cuda")
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    ops.gpu_qk_norm_rope(q, k, qn, kn, qo, ko, NQ, NKV, D, D, 0, None, 0, T, 1e6, 1e-6)
    inv_freq = torch.pow(torch.tensor(1e6, dtype=torch.float64, device="cuda"),
                         -2.0 * torch.arange(D // 2, device="cuda", dtype=torch.float64) / D)
    worst = 0.0
    for r in range(0, T, CH):
        for src, gam, dst, nh in ((q, qn, qo, NQ), (k, kn, ko, NKV)):
            v = src[r:r + CH].double().view(-1, nh, D)
            v = v * torch.rsqrt((v * v).mean(dim=2, keepdim=True) + 1e-6) * gam.double()
            pos = torch.arange(r, r + v.shape[0], device="cuda", dtype=torch.float64)
            ang = pos[:, None] * inv_freq[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            lo, hi = v[..., : D // 2], v[..., D // 2:]
            ref = torch.cat([lo * c - hi * s, lo * s + hi * c], dim=2)
            got = dst[r:r + CH].double().view(-1, nh, D)
            # row-relative error (rotated values cancel): bf16 rounding is 2^-9 of the value, here of the row maximum
            err = (got - ref).abs().amax(dim=2) / ref.abs().amax(dim=2)
            worst = max(worst, float(err.max()))
    assert worst <= 2.0 ** -8
    # positions given explicitly give the same bits as pos0 + t, and so do two shards
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    qo2, ko2 = torch.empty_like(q), torch.empty_like(k)
    h = T // 2 + 3
    ops.gpu_qk_norm_rope(q[:h], k[:h], qn, kn, qo2[:h], ko2[:h], NQ, NKV, D, D, 0, pos[:h], 0, h, 1e6, 1e-6)
    ops.gpu_qk_norm_rope(q[h:], k[h:], qn, kn, qo2[h:], ko2[h:], NQ, NKV, D, D, 0, None, h, T - h, 1e6, 1e-6)
    assert torch.equal(qo2.view(torch.int16), qo.view(torch.int16)) and torch.equal(ko2.view(torch.int16), ko.view(torch.int16))


def test_embed_full(ops):
    nb = E // 32
    g = torch.Generator(device="cuda").manual_seed(7)
    blocks = torch.empty(VOCAB * nb, 34, device="cuda", dtype=torch.uint8)
    d = (1e-3 + torch.rand(VOCAB * nb, device="cuda", generator=g) * 1.9e-2).half()
    blocks[:, 0:2] = d.view(torch.uint8).view(-1, 2)
    for r in range(0, VOCAB * nb, 1 << 22):
        n = min(1 << 22, VOCAB * nb - r)
        blocks[r:r + n, 2:] = torch.randint(-127, 128, (n, 32), device="cuda", generator=g, dtype=torch.int8).view(torch.uint8)
    ids = torch.randint(0, VOCAB, (T,), device="cuda", generator=g, dtype=torch.int32)
    ids[:3] = torch.tensor([0, VOCAB - 1, VOCAB // 2], dtype=torch.int32)
    out = torch.empty(T, E, device="cuda", dtype=bf)
    bad = ops.gpu_embed_rows(ops.QT_Q8_0, blocks.view(-1), nb * 34, VOCAB, ids, out, E, T)
    torch.cuda.synchronize()
    assert int(bad.item()) == 2**31 - 1
    tab = blocks.view(VOCAB, nb, 34)
    for r in range(0, T, CH):
        rows = tab[ids[r:r + CH].long()]                                   # [c][nb][34]
        scale = rows[:, :, 0:2].contiguous().view(torch.float16).float()    # [c][nb][1]
        vals = rows[:, :, 2:].contiguous().view(torch.int8).float() * scale
        assert torch.equal(out[r:r + CH].view(torch.int16), vals.view(-1, E).to(bf).view(torch.int16))


def test_moe_bookkeeping_full(ops):
    """The MoE configuration's bookkeeping at 262,144 tokens x 8 slots of 256 experts (2,097,152 entries): the router's
    selection against torch.topk, the grouping as a sorted permutation with exact tile bookkeeping, and the combine
    against a torch einsum, all rows."""
    n_expert, n_used, n = 256, 8, 512
    g = torch.Generator(device="cuda").manual_seed(11)
    logits = torch.randn(T, n_expert, device="cuda", generator=g) * 2
    ids = torch.empty(T, n_used, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, n_used, device="cuda")
    ops.gpu_moe_router(logits, None, None, ids, wts, None, n_expert, n_used, 0, T)
    p = torch.softmax(logits.double(), dim=1)
    top = torch.topk(p, n_used, dim=1)
    same = (ids.long() == top.indices)
    # (two probabilities that differ in double can round to one float, where the kernel's rule is the lower index)
    assert same.all(dim=1).float().mean() > 0.9999
    rows = same.all(dim=1)
    ref_w = (top.values / top.values.sum(dim=1, keepdim=True)).float()
    assert (wts[rows] - ref_w[rows]).abs().max() <= 2e-6
    assert torch.allclose(wts.sum(dim=1), torch.ones(T, device="cuda"), atol=1e-5)

    m = T * n_used
    tile = 128
    tok, pair = (torch.full((m,), -1, dtype=torch.int32, device="cuda") for _ in range(2))
    mt = ops.gpu_moe_max_tiles(T, n_used, n_expert, tile)
    ntl, te, ts, tn = (torch.zeros(k, dtype=torch.int32, device="cuda") for k in (1, mt, mt, mt))
    ops.gpu_moe_group(ids, T, n_used, n_expert, tile, tok, pair, ntl, te, ts, tn)
    flat = ids.reshape(-1).long()
    order = pair.long()
    assert torch.equal(torch.sort(order).values, torch.arange(m, device="cuda"))           # a permutation
    ex = flat[order]
    assert (ex[1:] >= ex[:-1]).all()                                                       # grouped by expert
    same_e = ex[1:] == ex[:-1]
    assert (order[1:][same_e] > order[:-1][same_e]).all()                                  # ascending inside a run
    assert torch.equal(tok.long(), order // n_used)
    counts = torch.bincount(flat, minlength=n_expert)
    k = int(ntl.item())
    assert k == int(((counts + tile - 1) // tile).sum()) <= mt
    assert torch.equal(torch.bincount(te[:k].long(), weights=tn[:k].double(), minlength=n_expert).long(), counts)
    starts = torch.cumsum(counts, 0) - counts
    first = torch.ones(k, dtype=torch.bool, device="cuda")
    first[1:] = te[1:k] != te[:k - 1]
    assert torch.equal(ts[:k][first].long(), starts[te[:k][first].long()])
    assert (tn[:k] >= 1).all() and (tn[:k] <= tile).all()

    down = torch.empty(T, n_used, n, device="cuda")
    for r in range(0, T, CH):
        down[r:r + CH] = torch.randn(CH, n_used, n, device="cuda", generator=g)
    out = torch.empty(T, n, device="cuda")
    ops.gpu_moe_combine(down, wts, None, None, out, n_used, n, T)
    for r in range(0, T, CH):
        ref = torch.einsum("tu,tun->tn", wts[r:r + CH].double(), down[r:r + CH].double())
        assert (out[r:r + CH].double() - ref).abs().max() <= 2e-6


def test_kv_rows_full(ops):
    """K rows of the whole batch into a block-major cache (blocks of 256 positions, 2 layers): FP16 rows exact against
    torch's conversion, Q8_0 rows dequantised within half a step, every other byte of the cache untouched."""
    n_vals, shift, layers = NKV * D, 8, 2
    B = 1 << shift
    src = rand((T, n_vals), 21).float()
    for kq in (0, 1):
        stride = n_vals if kq == 0 else n_vals * 17 // 32
        bstride = 2 * layers * B * stride
        cache = torch.full(((T // B) * bstride,), 0x7B7B, dtype=torch.int16, device="cuda")
        if kq == 0:
            ops.gpu_kv_store_f16(src, cache.view(torch.float16), n_vals, None, 0, T, stride, shift, bstride)
        else:
            ops.gpu_kv_store_q(src, cache, n_vals, None, 0, T, stride, shift, bstride, 1)
        blocks = cache.view(T // B, 2 * layers, B, stride)
        assert (blocks[:, 1:] == 0x7B7B).all()                       # V of this layer and the other layer: untouched
        rows = blocks[:, 0].reshape(T, stride)
        if kq == 0:
            assert torch.equal(rows.view(torch.float16), src.half())
        else:
            b8 = rows.contiguous().view(torch.int8)
            q = b8[:, :n_vals].float().view(T, n_vals // 32, 32)
            d = b8[:, n_vals:n_vals + n_vals // 16].contiguous().view(torch.float16).float()
            amax = src.view(T, n_vals // 32, 32).abs().amax(dim=2)
            assert torch.equal(d, (amax / 127).half().float())
            err = (q * (amax / 127).unsqueeze(2) - src.view(T, n_vals // 32, 32)).abs()
            assert (err <= (amax / 127).unsqueeze(2) * 0.5001 + 1e-12).all()
            assert (b8[:, n_vals + n_vals // 16:] == 0x7B).all()    # (no padding in these rows: empty slice)


def test_norm_chain_full(ops):
    """gemma_attn_post over the whole batch (n = 4096) against the separate launchers it fuses, bit for bit, and
    against a double-precision torch evaluation."""
    n = 4096
    g = torch.Generator(device="cuda").manual_seed(31)
    x, a = (torch.empty(T, n, device="cuda") for _ in range(2))
    for r in range(0, T, CH):
        x[r:r + CH] = torch.randn(CH, n, device="cuda", generator=g)
        a[r:r + CH] = torch.randn(CH, n, device="cuda", generator=g) * 2
    w_a, w1 = (1 + 0.1 * torch.randn(n, device="cuda", generator=g) for _ in range(2))
    x_out, y1 = torch.empty_like(x), torch.empty_like(x)
    ops.gpu_gemma_attn_post(x, a, w_a, x_out, w1, y1, None, None, n, T, 1e-6)
    sx = torch.empty_like(x)
    ops.gpu_add_normed(x, a, w_a, None, sx, n, T, 1e-6)
    assert torch.equal(sx, x_out)
    del sx
    worst = 0.0
    for r in range(0, T, CH):
        ad = a[r:r + CH].double()
        ref_x = x[r:r + CH].double() + ad * torch.rsqrt((ad * ad).mean(dim=1, keepdim=True) + 1e-6) * w_a.double()
        ref_y = ref_x * torch.rsqrt((ref_x * ref_x).mean(dim=1, keepdim=True) + 1e-6) * w1.double()
        worst = max(worst, float(((x_out[r:r + CH].double() - ref_x).abs().amax(dim=1) / ref_x.abs().amax(dim=1)).max()),
                    float(((y1[r:r + CH].double() - ref_y).abs().amax(dim=1) / ref_y.abs().amax(dim=1)).max()))
    assert worst <= 1e-6
