"""Per-launcher microbenchmark of the entry points around the hot path (the rows bench.py's sweep does not time):
MoE grouping / combine, strided SwiGLU / GEGLU, the Gemma-4 norm chains, KV-cache row writes (FP16, Q8_0, Q4_0, with
the Hadamard rotation), the 16-bit and int8 side outputs, the soft cap.

    python bench.py --micro [--tokens 65536] [--width 4096] [--iters 10] [--only REGEX]      (or: python microbench.py ...)

One line per case: CUDA-event time per launch (after 3 warm-ups; every case streams more bytes than the 126 MB L2
holds), the ALGORITHMIC bytes of the case (each input read once, each output written once, stated per case below),
GB/s, and that as a fraction of the copy bandwidth in MEASURED_PEAKS.json (repo root) when the file is there.
The timed calls are the library's launchers through ctypes; nothing here computes a result another way.
"""
import argparse
import json
import os
import re
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
import rocm_hip_b200 as m  # noqa: E402


def measured_copy_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return None


def time_launch(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3   # seconds per launch


def cases(T, n):
    """Yields (name, callable, algorithmic bytes per launch). fp32 rows [T][n] unless the name says otherwise."""
    R = lambda *s: torch.randn(*s, device="cuda")
    V = T * n
    x, a, o1, o2, o3 = R(T, n), R(T, n), R(T, n), R(T, n), R(T, n)
    w, w1, w2, w3 = R(n), R(n), R(n), R(n)
    sc = torch.tensor([0.7], device="cuda")
    # what the memory system gives plain library kernels at different read : write mixes (the denominators' context)
    yield "torch copy_ (read 1 : write 1)", lambda: o1.copy_(x), 8 * V
    yield "torch add (read 2 : write 1)", lambda: torch.add(x, a, out=o1), 12 * V
    yield "torch sum (read only)", lambda: x.sum(), 4 * V
    yield "torch zero_ (write only)", lambda: o1.zero_(), 4 * V
    # norm chains: inputs + outputs, 4 bytes each per value
    yield "add_normed", lambda: m.gpu_add_normed(x, a, w, sc, o1, n, T, 1e-6), 12 * V
    yield "gemma_attn_post", lambda: m.gpu_gemma_attn_post(x, a, w, o1, w1, o2, None, None, n, T, 1e-6), 16 * V
    yield "gemma_attn_post + router norm", lambda: m.gpu_gemma_attn_post(x, a, w, o1, w1, o2, w2, o3, n, T, 1e-6), 20 * V
    # MoE: 8 experts per token; down [T/8][8][n] so that the case stays the size of the others
    U, Tm, E = 8, max(T // 8, 1), 128
    down = R(Tm, U, n)
    wts = torch.rand(Tm, U, device="cuda")
    ids = torch.randint(0, E, (Tm, U), device="cuda", dtype=torch.int32)
    es = torch.rand(E, device="cuda") + 0.5
    xm, mlp, om1, om2 = R(Tm, n), R(Tm, n), R(Tm, n), R(Tm, n)
    yield "moe_combine (8 slots)", lambda: m.gpu_moe_combine(down, wts, None, None, om1, U, n, Tm), 4 * (U + 1) * Tm * n
    yield "moe_combine_scaled + shared", lambda: m.gpu_moe_combine(down, wts, xm, torch.rand(Tm, device="cuda"), om1, U, n, Tm, ids, es), 4 * (U + 2) * Tm * n
    yield "gemma_ffn_post (8 slots)", lambda: m.gpu_gemma_ffn_post(xm, mlp, down, wts, ids, es, U, w, w1, w2, sc, om1, w3, om2, n, Tm, 1e-6), 4 * (U + 4) * Tm * n
    # moe_group: ids in, two row lists out (12 bytes per entry): 6 MB, latency-bound by nature
    Tg = min(T, 65536)
    gi = torch.randint(0, E, (Tg, U), device="cuda", dtype=torch.int32)
    tok, pair = (torch.empty(Tg * U, device="cuda", dtype=torch.int32) for _ in range(2))
    mt = m.gpu_moe_max_tiles(Tg, U, E, 64)
    nt = torch.zeros(1, device="cuda", dtype=torch.int32)
    te, ts, tn = (torch.empty(mt, device="cuda", dtype=torch.int32) for _ in range(3))
    yield "moe_group (%d x 8 entries)" % Tg, lambda: m.gpu_moe_group(gi, Tg, U, E, 64, tok, pair, nt, te, ts, tn), 12 * Tg * U
    # embedding gather, bf16 rows of 5120 out: 4 (id) + row bytes + 2 * 5120 per token
    from rocm_hip_b200 import synth
    Ee, vocab = 5120, 32768
    eid = torch.randint(0, vocab, (T,), device="cuda", dtype=torch.int32)
    eout = torch.empty(T, Ee, device="cuda", dtype=torch.bfloat16)
    for qn in ("QT_Q8_0", "QT_Q4_0", "QT_Q4_K", "QT_Q6_K", "QT_Q5_1", "QT_F16"):
        qt = getattr(m, qn)
        rb = m.qt_row_size(qt, Ee)
        tab = torch.from_numpy(synth.gguf_table(0, "mb." + qn, qt, 64, Ee)).cuda().repeat(vocab // 64, 1).contiguous()
        yield "embed_rows %s -> bf16" % qn[3:], (lambda qt=qt, rb=rb, tab=tab: m.gpu_embed_rows(qt, tab, rb, vocab, eid, eout, Ee, T)), T * (4 + rb + 2 * Ee)
    # routers: logits [T][256] in, 8 ids + 8 weights out; with the shared-expert gate the x row is read too
    lg = R(T, 256)
    rid = torch.empty(T, 8, device="cuda", dtype=torch.int32)
    rw, rsg = torch.empty(T, 8, device="cuda"), torch.empty(T, device="cuda")
    rb = torch.zeros(256, device="cuda")
    yield "moe_router softmax (256 experts, top 8)", lambda: m.gpu_moe_router(lg, None, None, rid, rw, None, 256, 8, 0, T), T * (256 * 4 + 64)
    yield "moe_router softmax + shared gate", lambda: m.gpu_moe_router(lg, x, w, rid, rw, rsg, 256, 8, n, T), T * (256 * 4 + 68 + 4 * n)
    yield "moe_router sigmoid (256 experts, top 8)", lambda: m.gpu_moe_router_sigmoid(lg, rb, rid, rw, 256, 8, 1, 2.5, T), T * (256 * 4 + 64)
    yield "relu2", lambda: m.gpu_relu2(x, o1, T, n, n), 8 * V
    # gated activations on rows, 12 bytes per value
    gu = R(T, 2 * n)
    yield "swiglu flat", lambda: m.gpu_swiglu(x, a, o1, V), 12 * V
    yield "swiglu rows [gate|up] fused", lambda: m.gpu_swiglu_rows(gu, gu[:, n:], o1, T, n, 2 * n, 2 * n), 12 * V
    yield "geglu", lambda: m.gpu_geglu(x, a, o1, T, n, n, n), 12 * V
    yield "geglu rows [gate|up] fused", lambda: m.gpu_geglu(gu, gu[:, n:], o1, T, n, 2 * n, 2 * n), 12 * V
    yield "softcap (in place)", lambda: m.gpu_softcap(x, V, 30.0), 8 * V
    # side outputs: the producer's own traffic + 2 bytes (xh), or + a pass of 4 read + ~2.5 written (int8 formats)
    qx = m.Q8Buffers(V, "cuda", xh="bf16", int8=False)
    qa = m.Q8Buffers(V, "cuda", xh="bf16")
    yield "rmsnorm", lambda: m.gpu_add_rmsnorm(x, None, None, w, o1, n, T, 1e-6), 8 * V
    yield "rmsnorm + bf16 copy (one launch)", lambda: m.gpu_add_rmsnorm(x, None, None, w, o1, n, T, 1e-6, q8=qx), 10 * V
    yield "add+rmsnorm + bf16 copy (one launch)", lambda: m.gpu_add_rmsnorm(x, a, o2, w, o1, n, T, 1e-6, q8=qx), 18 * V
    yield "swiglu + bf16 copy (one launch)", lambda: m.gpu_swiglu(x, a, o1, V, q8=qx), 14 * V
    # int8 formats written by the producer itself (one launch): + 1 (q0) + 1 (qK) + ~0.53 (scales, sums) bytes per value
    yield "rmsnorm + bf16 copy + Q8_0/Q8_K (one launch)", lambda: m.gpu_add_rmsnorm(x, None, None, w, o1, n, T, 1e-6, q8=qa), (10 + 2.53) * V
    yield "add+rmsnorm + bf16 copy + Q8_0/Q8_K (one launch)", lambda: m.gpu_add_rmsnorm(x, a, o2, w, o1, n, T, 1e-6, q8=qa), (18 + 2.53) * V
    yield "swiglu + bf16 copy + Q8_0/Q8_K (one launch)", lambda: m.gpu_swiglu(x, a, o1, V, q8=qa), (14 + 2.53) * V
    # q/k norm + RoPE (bf16, 40 + 8 heads of 128): 2 bytes in and out per value; with the K heads written to the cache
    nq, nkv, D = 40, 8, 128
    qb, kb = R(T, nq * D).bfloat16(), R(T, nkv * D).bfloat16()
    qo, ko = torch.empty_like(qb), torch.empty_like(kb)
    qn, kn = 1 + 0.1 * R(D), 1 + 0.1 * R(D)
    kc = torch.zeros(T * nkv * D, device="cuda", dtype=torch.float16)
    ct, st2 = torch.empty(T, D // 2, device="cuda"), torch.empty(T, D // 2, device="cuda")
    yield "rope_table (64 pairs per token)", lambda: m.gpu_rope_table(None, 0, T, D, 0, 1e6, ct, st2), 8 * T * (D // 2)
    yield "qk_norm_rope_tab (bf16, tables read)", lambda: m.gpu_qk_norm_rope_tab(qb, kb, qn, kn, qo, ko, nq, nkv, D, D, ct, st2, T, 1e-6), 4 * T * (nq + nkv) * D
    yield "qk_norm_rope (bf16)", lambda: m.gpu_qk_norm_rope(qb, kb, qn, kn, qo, ko, nq, nkv, D, D, 0, None, 0, T, 1e6, 1e-6), 4 * T * (nq + nkv) * D
    yield "qk_norm_rope_kv (bf16, K into the fp16 cache)", lambda: m.gpu_qk_norm_rope_kv(qb, kb, qn, kn, qo, kc, nkv * D, 30, 0, nq, nkv, D, D, 0, None, 0, T, 1e6, 1e-6), 4 * T * (nq + nkv) * D
    yield "qk_norm_rope_tab_kv (bf16, tables read, K into the fp16 cache)", lambda: m.gpu_qk_norm_rope_tab_kv(qb, kb, qn, kn, qo, kc, nkv * D, 30, 0, nq, nkv, D, D, ct, st2, None, 0, T, 1e-6), 4 * T * (nq + nkv) * D
    yield "qk_norm_rope + kv_store_f16 (two launches)", lambda: (m.gpu_qk_norm_rope(qb, kb, qn, kn, qo, ko, nq, nkv, D, D, 0, None, 0, T, 1e6, 1e-6), m.gpu_kv_store_f16(ko, kc, nkv * D, None, 0, T, nkv * D, 30, 0)), 4 * T * (nq + nkv) * D + 4 * T * nkv * D
    # KV rows: 1024 values per token row (8 heads x 128), 4 T rows
    nv, Tk = 1024, 4 * T
    src = R(Tk, nv)
    sb = src.to(torch.bfloat16)
    c16 = torch.zeros(Tk * nv, device="cuda", dtype=torch.float16)
    yield "kv_store_f16", lambda: m.gpu_kv_store_f16(src, c16, nv, None, 0, Tk, nv, 30, 0), 6 * Tk * nv
    yield "kv_store_f16 (bf16 rows)", lambda: m.gpu_kv_store_f16(sb, c16, nv, None, 0, Tk, nv, 30, 0), 4 * Tk * nv
    for kq, name, st in ((1, "q8_0", nv * 17 // 32), (2, "q4_0", nv * 9 // 32)):
        c = torch.zeros(Tk * st, device="cuda", dtype=torch.int16)
        yield "kv_store_%s" % name, (lambda c=c, st=st, kq=kq: m.gpu_kv_store_q(src, c, nv, None, 0, Tk, st, 30, 0, kq)), Tk * (4 * nv + 2 * st)
        yield "kv_store_%s rotated (128)" % name, (lambda c=c, st=st, kq=kq: m.gpu_kv_store_q(src, c, nv, None, 0, Tk, st, 30, 0, kq, rot_block=128)), Tk * (4 * nv + 2 * st)
        yield "kv_store_%s (bf16 rows)" % name, (lambda c=c, st=st, kq=kq: m.gpu_kv_store_q(sb, c, nv, None, 0, Tk, st, 30, 0, kq)), Tk * (2 * nv + 2 * st)
    yield "hadamard_rot (128)", lambda: m.gpu_hadamard_rot(src, src, Tk * 8, 128, 128), 8 * Tk * nv
    yield "hadamard_rot (512)", lambda: m.gpu_hadamard_rot(src, src, Tk * 2, 512, 512), 8 * Tk * nv


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--width", type=int, default=4096, help="row width n (a multiple of 256, at most 4096)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default=None, help="regular expression on the case name")
    ap.add_argument("--once", action="store_true",
                    help="launch every selected case exactly once and time nothing (the run a profiler capture wraps)")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    assert m.gpu_ops_init("gpu_ops.co") == 0
    peak = measured_copy_peak()
    print("%-50s %10s %10s %9s %s" % ("case", "us", "MB", "GB/s", "of measured copy peak" if peak else ""))
    for name, fn, nbytes in cases(args.tokens, args.width):
        if args.only and not re.search(args.only, name):
            continue
        if args.once:
            fn()
            torch.cuda.synchronize()
            print("%-50s launched once" % name)
            continue
        sec = time_launch(fn, args.iters)
        gbs = nbytes / sec / 1e9
        print("%-50s %10.1f %10.1f %9.0f %s" % (name, sec * 1e6, nbytes / 1e6, gbs, "%.3f" % (gbs / peak) if peak else ""))


if __name__ == "__main__":
    main()
