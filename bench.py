#!/usr/bin/env python
"""Benchmark of the fused layer-op path. One sweep = one pass of the layer's ops over one batch of synthetic rows
(embedding gather -> RMSNorm -> cos/sin table -> q/k norm + RoPE -> residual add + RMSNorm -> SwiGLU -> residual add +
RMSNorm), in the order a layer of the reference's forward pass issues them (src/qwen_model.cpp:980-990, 941-957). One
step = `sweeps_per_step` sweeps back to back (as many as keep a step near 30 ms whatever the GPU count, so that the
timed region of K steps is long enough for the clock samples to mean something).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c5|c4|c3|c2|c1] [--impl reference]

For N > 1 launch one process per GPU with torch.distributed.run; rows are sharded by token, no collective touches
the data path (torch.distributed only carries the barrier and the max over ranks of the device-timed duration).
Prints ONE JSON line on rank 0:
  value       token rows per second through the whole sweep, inputs resident in HBM, all ranks together
  kernels     per kernel: rows/s, algorithmic GB/s, fraction of the measured HBM copy peak and of the nominal 8 TB/s
  roofline    the dominant kernel (SwiGLU) against the measured HBM peak
  configs     the same per-kernel table for the other workloads (c1 .. c4), each kernel launched on cold inputs
  e2e         the same sweep through the host-buffer C-ABI call, host<->device copies inside the timed region, next to
              the time the same bytes take as plain copies
  cpu_baseline the reference's CPU functions (or their restatement) on the host cores, on a bounded row sample
--impl reference times that CPU path alone with all host threads and prints the same line shape.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0

# Workloads: row counts and widths of the five benchmark configurations. c5 is the headline multi-GPU configuration.
WORKLOADS = {
    "c5": dict(name="dense-27B-shape layer-op sweep", dtype="bf16", T=262144, E=5120, n_q=40, n_kv=8, D=128,
               n_rot=128, theta=1e6, FF=17408, qtype=8, vocab=151936, eps=1e-6),
    "c3": dict(name="Qwen3.5-4B-like prefill layer-op sweep", dtype="bf16", T=16384, E=2560, n_q=16, n_kv=4, D=256,
               n_rot=64, theta=1e7, FF=9216, qtype=2, vocab=248320, eps=1e-6, gated=1),
    "c4": dict(name="MoE-shape expert-grouped SwiGLU + RMSNorm", dtype="bf16", T=65536, E=2048, n_q=0, n_kv=0, D=0,
               n_rot=0, theta=1e6, FF=8 * 512, qtype=0, vocab=0, eps=1e-6, moe=1),
    "c2": dict(name="decode-shape layer ops, 64 sequences x 1 token (latency-bound)", dtype="bf16", T=64, E=1024, n_q=16,
               n_kv=8, D=128, n_rot=128, theta=1e6, FF=3072, qtype=8, vocab=151936, eps=1e-6, random_positions=32768),
    "c1": dict(name="Qwen3-0.6B-shape layer ops", dtype="f32", T=2427, E=1024, n_q=16, n_kv=8, D=128, n_rot=128,
               theta=1e6, FF=3072, qtype=8, vocab=151936, eps=1e-6),
}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


from rocm_hip_b200.sharding import shard  # noqa: E402  (contiguous row range of a rank)


def dram_traffic_ratio(kernel):
    """DRAM bytes per algorithmic byte of a kernel, from the tracked summary of its profiler capture (a small case;
    every byte is touched once, so traffic grows with the rows). Returns (ratio or None, where it came from)."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        e = json.load(open(p))[kernel]
        return float(e["dram_bytes"]) / float(e["algorithmic_bytes"]), f"profiles/dram_traffic.json[{kernel}]: {e['capture']}"
    except Exception:
        return None, "no capture on file"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi every 10 ms. It is started ahead of the warm-up (the tool
    takes a moment to come up); mark() brackets the timed region and only samples taken inside it are reported (the
    nearest ones if the region was shorter than a sampling interval)."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.t0, self.t1 = index, None, None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "10"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), [n for n, v in zip(names, f[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if self.t0 is not None and self.t0 <= r[0] <= self.t1]
        if not inside and rows and self.t0 is not None:   # region shorter than an interval: the two nearest samples
            mid = 0.5 * (self.t0 + self.t1)
            inside = sorted(rows, key=lambda r: abs(r[0] - mid))[:2]
        if not inside:
            inside = rows
        sm = [r[1] for r in inside]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(r[2] for r in inside) if inside else None,
                "reasons": sorted({n for r in inside for n in r[3]}), "samples": len(inside)}


# ------------------------------------------------------------------------------------------------ device workload

class Sweep:
    """Device-resident synthetic inputs of one rank's rows and the list of kernels of one step."""

    def __init__(self, wl, T, row0, device, seed=0):
        import torch
        import rocm_hip_b200 as ops
        self.torch, self.ops, self.wl, self.T = torch, ops, wl, T
        self.dt = torch.bfloat16 if wl["dtype"] == "bf16" else torch.float32
        s = self.s = 2 if wl["dtype"] == "bf16" else 4
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + row0 + 17)
        E, FF = wl["E"], wl["FF"]
        randn = lambda *shape: torch.randn(*shape, device=device, generator=g, dtype=torch.float32).to(self.dt)
        big = lambda rows, cols: torch.cat([randn(min(8192, rows - r), cols) for r in range(0, rows, 8192)])
        self.w1 = (1 + 0.1 * torch.randn(E, device=device, generator=g)).float()
        self.w2 = (1 + 0.1 * torch.randn(E, device=device, generator=g)).float()
        self.kernels = []   # (name, callable, algorithmic bytes, rows, unit rows name)
        self.x = torch.empty(T, E, device=device, dtype=self.dt)
        self.x_alt = torch.empty_like(self.x)
        self.xn = torch.empty_like(self.x)
        if wl.get("moe"):
            # 65,536 tokens x hidden 2048 through RMSNorm; top-8 of 256 experts, rows grouped by expert id: the
            # grouped (token, slot) rows of width 512 are what SwiGLU sees. Grouping permutes rows; the map is flat.
            self.x.copy_(big(T, E))
            rows = T * 8
            self.g, self.u = big(rows, 512), big(rows, 512)
            self.act = torch.empty_like(self.g)
            self.kernels.append(("rmsnorm", lambda: ops.gpu_add_rmsnorm(self.x, None, self.x, self.w1, self.xn, E, T, wl["eps"]),
                                 T * 2 * E * s + 4 * E, T, "token rows"))
            self.kernels.append(("swiglu_expert_rows", lambda: ops.gpu_swiglu(self.g, self.u, self.act, rows * 512),
                                 rows * 3 * 512 * s, rows, "expert rows"))
            self.dominant = "swiglu_expert_rows"
            return
        nq, nkv, D = wl["n_q"], wl["n_kv"], wl["D"]
        gated = wl.get("gated", 0)
        qs = 2 * D if gated else D
        vocab, qt = wl["vocab"], wl["qtype"]
        nb = E // 32
        bb = 34 if qt == 8 else 18
        self.row_bytes = nb * bb
        # quantised table: fp16 scale ~ U(1e-3, 2e-2) then the payload (int8 in [-127,127] / nibbles in [0,15])
        blocks = torch.empty(vocab * nb, bb, device=device, dtype=torch.uint8)
        d = (1e-3 + torch.rand(vocab * nb, device=device, generator=g) * (2e-2 - 1e-3)).half()
        blocks[:, 0:2] = d.view(torch.uint8).view(-1, 2)
        for r in range(0, vocab * nb, 1 << 22):
            n = min(1 << 22, vocab * nb - r)
            if qt == 8:
                blocks[r:r + n, 2:] = torch.randint(-127, 128, (n, 32), device=device, generator=g, dtype=torch.int8).view(torch.uint8)
            else:
                blocks[r:r + n, 2:] = torch.randint(0, 256, (n, 16), device=device, generator=g, dtype=torch.int16).to(torch.uint8)
        self.table = blocks.view(-1)
        del d
        self.ids = torch.randint(0, vocab, (T,), device=device, generator=g, dtype=torch.int32)
        self.bad = torch.full((1,), 2**31 - 1, dtype=torch.int32, device=device)
        self.pos0 = row0
        self.positions = None
        if wl.get("random_positions"):   # one token per sequence, each at its own position
            self.positions = torch.randint(0, wl["random_positions"], (T,), device=device, generator=g, dtype=torch.int32)
        self.q = big(T, nq * qs)
        self.k = big(T, nkv * D)
        self.q_out = torch.empty(T, nq * D, device=device, dtype=self.dt)
        self.k_out = torch.empty(T, nkv * D, device=device, dtype=self.dt)
        half = wl["n_rot"] // 2
        self.cos_tab = torch.empty(T, half, device=device)
        self.sin_tab = torch.empty(T, half, device=device)
        self.qn = (1 + 0.1 * torch.randn(D, device=device, generator=g)).float()
        self.kn = (1 + 0.1 * torch.randn(D, device=device, generator=g)).float()
        self.proj1 = big(T, E)
        self.proj2 = big(T, E)
        self.g, self.u = big(T, FF), big(T, FF)
        self.act = torch.empty_like(self.g)
        eps = wl["eps"]
        K = self.kernels
        K.append(("embed_gather", lambda: ops.gpu_embed_rows(qt, self.table, self.row_bytes, vocab, self.ids, self.x, E, T, 1.0, self.bad),
                  T * (4 + self.row_bytes + E * s), T, "token rows"))
        K.append(("rmsnorm", lambda: ops.gpu_add_rmsnorm(self.x, None, self.x, self.w1, self.xn, E, T, eps),
                  T * 2 * E * s + 4 * E, T, "token rows"))
        # The cos / sin of the tokens' angles are computed once (a forward pass does it once for all its layers; here
        # once per sweep, its time counted in the step) and the q/k kernel reads them. The table is not algorithmic
        # traffic of the q/k kernel: its bytes are the head rows in and out.
        K.append(("rope_table", lambda: ops.gpu_rope_table(self.positions, self.pos0, T, wl["n_rot"], 0, wl["theta"], self.cos_tab,
                                                            self.sin_tab),
                  T * 4 * (1 if self.positions is not None else 0) + T * half * 8, T, "token rows"))
        K.append(("qk_norm_rope", lambda: ops.gpu_qk_norm_rope_tab(self.q, self.k, self.qn, self.kn, self.q_out, self.k_out, nq,
                                                                   nkv, D, wl["n_rot"], self.cos_tab, self.sin_tab, T, eps, gated, 1),
                  T * ((nq * qs if not gated else nq * D) + nkv * D + (nq + nkv) * D) * s, T * (nq + nkv), "head rows"))
        K.append(("add_rmsnorm_ffn", lambda: ops.gpu_add_rmsnorm(self.x, self.proj1, self.x_alt, self.w2, self.xn, E, T, eps),
                  T * 4 * E * s + 4 * E, T, "token rows"))
        K.append(("swiglu", lambda: ops.gpu_swiglu(self.g, self.u, self.act, T * FF), T * 3 * FF * s, T, "token rows"))
        K.append(("add_rmsnorm_next", lambda: ops.gpu_add_rmsnorm(self.x_alt, self.proj2, self.x, self.w1, self.xn, E, T, eps),
                  T * 4 * E * s + 4 * E, T, "token rows"))
        self.dominant = "swiglu"

    def step(self, events=None, flush=None):
        """One sweep. events: per kernel a (start, end) pair recorded around its launch. flush: a tensor larger than L2
        that is rewritten before every kernel (outside the event pair), for workloads whose tensors would otherwise
        still sit in the 126 MB L2 from the kernel that produced them."""
        for i, (_, fn, _, _, _) in enumerate(self.kernels):
            if flush is not None:
                flush.add_(1)
            if events is not None:
                events[i][0].record()
            fn()
            if events is not None:
                events[i][1].record()


# ------------------------------------------------------------------------------------------------ host-buffer e2e

class HostSweep:
    """The same sweep through the host-buffer C-ABI call (b200_host_layer_sweep; the MoE workload, which has no gather
    or q/k step, through b200_host_add_rmsnorm + b200_host_swiglu): every true input starts in page-locked host memory
    and every result ends there, each step; the residual stream between the ops stays on the device, as the
    reference keeps it in place (s.x / s.x_alt, src/qwen_model.cpp:946-957)."""

    def __init__(self, wl, T, row0, table_dev, row_bytes, slot_bytes=256 << 20, n_slots=4):
        import torch
        import rocm_hip_b200 as ops
        self.wl, self.T, self.ops = wl, T, ops
        dt = torch.bfloat16 if wl["dtype"] == "bf16" else torch.float32
        s = 2 if wl["dtype"] == "bf16" else 4
        E, FF = wl["E"], wl["FF"]
        g = torch.Generator().manual_seed(4242 + row0)
        pin = lambda *shape, dtype=dt: torch.empty(*shape, dtype=dtype).pin_memory()
        rnd = lambda *shape: pin(*shape).copy_(torch.randn(*shape, generator=g).to(dt))
        self.host = ops.HostRows(slot_bytes=slot_bytes, n_slots=n_slots)
        self.w = (1 + 0.1 * torch.randn(E, generator=g)).float()
        self.calls = []
        H = self.host
        if wl.get("moe"):
            rows = T * 8
            x, xn = rnd(T, E), pin(T, E)
            gg, uu, act = rnd(rows, 512), rnd(rows, 512), pin(rows, 512)
            self.calls.append(lambda: H.add_rmsnorm(x, None, None, self.w, xn, E, T, wl["eps"]))
            self.calls.append(lambda: H.swiglu(gg, uu, act, rows, 512))
            self.inputs, self.outputs = [x, gg, uu], [xn, act]
        else:
            nq, nkv, D = wl["n_q"], wl["n_kv"], wl["D"]
            gated = wl.get("gated", 0)
            qs = 2 * D if gated else D
            ids = pin(T, dtype=torch.int32).copy_(torch.randint(0, wl["vocab"], (T,), generator=g, dtype=torch.int32))
            q, k = rnd(T, nq * qs), rnd(T, nkv * D)
            p1, p2, gg, uu = rnd(T, E), rnd(T, E), rnd(T, FF), rnd(T, FF)
            xn1, qo, ko, xn2, act, xo, xn3 = pin(T, E), pin(T, nq * D), pin(T, nkv * D), pin(T, E), pin(T, FF), pin(T, E), pin(T, E)
            qn = (1 + 0.1 * torch.randn(D, generator=g)).float()
            kn = (1 + 0.1 * torch.randn(D, generator=g)).float()
            self.calls.append(lambda: H.layer_sweep(
                qtype=wl["qtype"], table_dev=table_dev, row_bytes=row_bytes, vocab=wl["vocab"], tokens=ids, E=E,
                w_attn_norm=self.w, w_ffn_norm=self.w, w_next_norm=self.w, eps=wl["eps"], xn_attn=xn1, qfull=q, k=k, q_out=qo,
                k_out=ko, q_norm=qn, k_norm=kn, n_q=nq, n_kv=nkv, head_dim=D, n_rot=wl["n_rot"], freq_base=wl["theta"],
                attn_proj=p1, xn_ffn=xn2, gate=gg, up=uu, FF=FF, act=act, ffn_proj=p2, x_out=xo, xn_next=xn3, T=T, pos0=row0,
                gated=gated))
            self.inputs, self.outputs = [ids, q, k, p1, p2, gg, uu], [xn1, qo, ko, xn2, act, xo, xn3]
            self.keep = (qn, kn)
        self.h2d = sum(t.numel() * t.element_size() for t in self.inputs)
        self.d2h = sum(t.numel() * t.element_size() for t in self.outputs)

    def step(self):
        for c in self.calls:
            c()

    def copy_only_ms(self, steps):
        """The same bytes as plain copies and nothing else: every input tensor host -> device on one stream, every
        output tensor device -> host on another, both directions at once. The ceiling the host-buffer call is held to."""
        import torch
        dev_in = [torch.empty(t.shape, dtype=t.dtype, device="cuda") for t in self.inputs]
        dev_out = [torch.empty(t.shape, dtype=t.dtype, device="cuda") for t in self.outputs]
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def once():
            up.wait_stream(torch.cuda.current_stream())
            down.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(up):
                for d, h in zip(dev_in, self.inputs):
                    d.copy_(h, non_blocking=True)
            with torch.cuda.stream(down):
                for h, d in zip(self.outputs, dev_out):
                    h.copy_(d, non_blocking=True)
            torch.cuda.current_stream().wait_stream(up)
            torch.cuda.current_stream().wait_stream(down)
        once()
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            once()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps


# ------------------------------------------------------------------------------------------------ CPU baseline

class CpuSweep:
    """The sweep on the host cores with the reference's own CPU functions (oracle/_ref, built from the reference's
    qwen_ops.cpp / quant_types.cpp) when that build is present, else with their restatement (oracle/). fp32, the only
    precision the reference's CPU path has. This is the one place the benchmark executes anything under oracle/."""

    def __init__(self, wl, T, threads):
        import numpy as np
        from oracle import oracle as O
        from rocm_hip_b200 import synth
        self.np, self.O = np, O
        self.lib = O.ref() if O.have_ref() else O.port()
        self.kind = "reference" if O.have_ref() else "port"
        self.threads = threads or self.lib.cpu_hardware_threads()
        self.wl, self.T = wl, T
        E, FF = wl["E"], wl["FF"]
        rng = np.random.default_rng(0)
        f = lambda *shape: rng.standard_normal(shape, dtype=np.float32)
        self.w = (1 + 0.1 * rng.standard_normal(E)).astype(np.float32)
        self.x, self.x_alt, self.xn = np.empty((T, E), np.float32), np.empty((T, E), np.float32), np.empty((T, E), np.float32)
        if wl.get("moe"):
            self.x[:] = f(T, E)
            self.g, self.u = f(T * 8, 512), f(T * 8, 512)
            self.act = np.empty_like(self.g)
            return
        nq, nkv, D = wl["n_q"], wl["n_kv"], wl["D"]
        qs = 2 * D if wl.get("gated") else D
        vocab = min(wl["vocab"], 4096)   # a slice of the table: the gather's cost per row does not depend on the vocabulary
        self.vocab = vocab
        maker = synth.q8_0_table if wl["qtype"] == 8 else synth.q4_0_table
        self.table = maker(0, "bench.cpu.table", vocab, E)
        self.ids = rng.integers(0, vocab, T).astype(np.int32)
        self.q, self.k = f(T, nq * qs), f(T, nkv * D)
        self.qo, self.ko = np.empty((T, nq * D), np.float32), np.empty((T, nkv * D), np.float32)
        self.qn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
        self.kn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
        self.p1, self.p2 = f(T, E), f(T, E)
        self.g, self.u = f(T, FF), f(T, FF)
        self.act = np.empty_like(self.g)

    def step(self):
        L, p, wl, T, th = self.lib, self.O.ptr, self.wl, self.T, self.threads
        E, FF, eps = wl["E"], wl["FF"], wl["eps"]
        if wl.get("moe"):
            L.cpu_add_rmsnorm(p(self.x), None, None, p(self.w), p(self.xn), E, T, eps, th)
            L.cpu_swiglu(p(self.g), p(self.u), p(self.act), self.g.size, th)
            return
        st = L.cpu_embed_rows(wl["qtype"], p(self.table), self.table.shape[1], self.vocab, p(self.ids), p(self.x), E, T, 1.0, th)
        assert st == 0
        L.cpu_add_rmsnorm(p(self.x), None, None, p(self.w), p(self.xn), E, T, eps, th)
        L.cpu_qk_norm_rope(p(self.q), p(self.k), p(self.qn), p(self.kn), p(self.qo), p(self.ko), wl["n_q"], wl["n_kv"], wl["D"],
                           wl["n_rot"], None, 0, T, wl["theta"], eps, 1 if wl.get("gated") else 0, 1, th)
        L.cpu_add_rmsnorm(p(self.x), p(self.p1), p(self.x_alt), p(self.w), p(self.xn), E, T, eps, th)
        L.cpu_swiglu(p(self.g), p(self.u), p(self.act), self.g.size, th)
        L.cpu_add_rmsnorm(p(self.x_alt), p(self.p2), p(self.x), p(self.w), p(self.xn), E, T, eps, th)


def time_cpu(wl, T, steps, warmup, threads=0):
    cs = CpuSweep(wl, T, threads)
    for _ in range(warmup):
        cs.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        cs.step()
    dt = (time.perf_counter() - t0) / steps
    return cs, dt


def cpu_sample_rows(wl, budget_s):
    """Rows of the bounded CPU sample: calibrated on a short run so that one step costs about budget_s seconds."""
    probe = 256 if not wl.get("moe") else 1024
    _, dt = time_cpu(wl, probe, 1, 1)
    rows = int(probe * budget_s / max(dt, 1e-6))
    cap = 16384 if not wl.get("moe") else 65536
    return max(probe, min(rows, cap, wl["T"]))


def run_reference(args, wl, rank, world):
    if rank != 0:
        return
    rows = args.cpu_rows or cpu_sample_rows(wl, 2.0)
    cs, dt = time_cpu(wl, rows, args.steps, max(args.warmup, 1))
    val = rows / dt
    base = {"value": val, "unit": "rows/s", "cores": cs.threads, "kind": cs.kind,
            "sample": f"{rows} token rows of the {args.config} sweep per step, fp32 (the reference's CPU precision), all host threads"}
    line = {"impl": "reference", "metric": "layer-op sweep throughput (token rows/s)", "value": val, "unit": "rows/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.config}: {wl['name']}", "rows_per_step": rows}, "cpu_baseline": base,
            "e2e": {"value": val, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


_REAL_STDOUT = None


def claim_stdout():
    """Keeps stdout for the one JSON line: anything libraries print to file descriptor 1 (NCCL's version banner, for
    one) goes to stderr instead."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def kernel_table(sw, per_kernel_ms, world, peak, median=None, best=None):
    """Per kernel: mean launch time over the timed launches (ms; the figures derive from it), and their median and
    best, max over ranks each."""
    rows = []
    for i, ((name, _, nbytes, nrows, unit), ms) in enumerate(zip(sw.kernels, per_kernel_ms)):
        gbs = nbytes / (ms * 1e-3) / 1e9
        extra = {"ms_median": median[i], "ms_best": best[i]} if median and best else {}
        rows.append({"name": name, "ms": ms, **extra, "rows_per_s": nrows * world / (ms * 1e-3), "rows": unit,
                     "algorithmic_bytes_per_gpu": nbytes, "gbs_per_gpu": gbs, "gbs_all_gpus": gbs * world,
                     "frac_of_measured_peak": gbs / peak, "frac_of_8tbs": gbs / NOMINAL_HBM_GBS})
    return rows


def sweeps_per_step(wl, T):
    """Sweeps in one step: as many as bring a step's rows to about the rows of 3 sweeps of the full c5 batch on one
    GPU (~30 ms of device time, so that 20 steps time 0.6 s whatever the GPU count), from the rank's row count and
    row width alone."""
    per_row = wl["E"] * 8 + wl["FF"] * 3 + (wl["n_q"] + wl["n_kv"]) * wl["D"] * 2
    return max(1, min(4096, round(3 * 262144 * (5120 * 8 + 17408 * 3 + 48 * 128 * 2) / (T * per_row))))


def main():
    if "--micro" in sys.argv:   # the per-launcher table of the entry points around the sweep (microbench.py)
        sys.argv.remove("--micro")
        import microbench
        return microbench.main()
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="total token rows (default: the configuration's)")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: the configuration's rows are sharded over the GPUs; weak: every GPU gets all of them")
    ap.add_argument("--e2e-rows", type=int, default=16384, help="token rows per rank of the host-buffer measurement")
    ap.add_argument("--cpu-rows", type=int, default=0, help="token rows of the CPU sample (default: calibrated)")
    ap.add_argument("--sweeps-per-step", type=int, default=0, help="default: chosen from the rank's rows (see sweeps_per_step)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the per-kernel tables of the other workloads")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS[args.config]
    if args.impl == "reference":
        run_reference(args, wl, rank, world)
        return

    import torch
    import torch.distributed as dist
    import rocm_hip_b200 as ops

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)   # the harness's barrier and max-reduce only
    assert ops.gpu_ops_init("gpu_ops.co") == 0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor(v, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    peak, peak_src = measured_peak()

    def rank_rows(T_total):
        if args.scaling == "strong":
            lo, hi = shard(T_total, rank, world)
            return lo, hi - lo, T_total
        return rank * T_total, T_total, T_total * world

    def time_sweeps(sw, steps, reps, flush=None, clocks=None):
        """Times steps x reps sweeps between two barriers; returns (ms per step, ms per launch of each kernel), max over
        ranks. Every launch sits between its own pair of events."""
        nk = len(sw.kernels)
        ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nk)]
              for _ in range(steps * reps)]
        barrier()
        if clocks:
            clocks.mark_begin()
        start.record()
        for i in range(steps * reps):
            sw.step(ev[i], flush)
        end.record()
        barrier()
        if clocks:
            clocks.mark_end()
        times = [sorted(e[j][0].elapsed_time(e[j][1]) for e in ev) for j in range(nk)]
        per_kernel = [sum(t) / len(t) for t in times]
        red = max_over_ranks([start.elapsed_time(end) / steps] + per_kernel + [t[len(t) // 2] for t in times] + [t[0] for t in times])
        time_sweeps.median, time_sweeps.best = red[1 + nk:1 + 2 * nk], red[1 + 2 * nk:]
        return red[0], red[1:1 + nk]

    # ---- the headline workload
    lo, T, T_total = rank_rows(args.tokens or wl["T"])
    sw = Sweep(wl, T, lo, device)
    nk = len(sw.kernels)
    reps = args.sweeps_per_step or sweeps_per_step(wl, T)
    warm = max(args.warmup, 3)
    clocks = ClockSampler(local)
    clocks.start()
    for _ in range(warm):
        sw.step()
    launches0 = ops.launch_count()
    ms_step, per_kernel_ms = time_sweeps(sw, args.steps, reps, clocks=clocks)
    head_median, head_best = time_sweeps.median, time_sweeps.best
    clk = clocks.stop()
    launches = ops.launch_count() - launches0
    # A sweep of a few microseconds per kernel is bound by launch latency: it is also timed as replays of a CUDA graph
    # of one sweep, which takes the host's launch cost out; that time becomes the step's.
    graph_ms = None
    if ms_step / reps < 1.0:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            sw.step()
            with torch.cuda.graph(g, stream=side):
                sw.step()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            g.replay()
        barrier()
        start.record()
        for _ in range(args.steps * reps):
            g.replay()
        end.record()
        barrier()
        launches += nk * args.steps * reps
        graph_ms = max_over_ranks([start.elapsed_time(end)])[0] / args.steps
        ms_step = graph_ms
    if not wl.get("moe"):
        assert int(sw.bad.item()) == 2**31 - 1
    kernels = kernel_table(sw, per_kernel_ms, world, peak, head_median, head_best)
    dom = next(k for k in kernels if k["name"] == sw.dominant)
    ratio, ratio_src = dram_traffic_ratio("swiglu_bf16" if wl["dtype"] == "bf16" else "swiglu_f32")
    roof = {"kernel": dom["name"], "bound": "hbm", "achieved": dom["gbs_per_gpu"], "peak": peak, "unit": "GB/s",
            "frac": dom["gbs_per_gpu"] / peak, "traffic": ratio * dom["algorithmic_bytes_per_gpu"] if ratio else None,
            "traffic_source": ratio_src, "peak_source": f"of {peak_src}",
            "algorithmic_bytes_per_launch": dom["algorithmic_bytes_per_gpu"], "ms_per_launch": dom["ms"]}
    cache_note = ("every tensor of a sweep is larger than L2 (126 MB); no flush needed" if T * wl["E"] * sw_bytes(wl) > 126e6
                  else "tensors near or below the L2 size: warm from the producing kernel, as in a forward pass")
    table_dev, row_bytes = getattr(sw, "table", None), getattr(sw, "row_bytes", 0)

    # ---- end to end through the host-buffer call
    e2e, launches_e2e = None, 0
    if not args.no_e2e:
        Te = min(args.e2e_rows, T)
        l0 = ops.launch_count()
        hs = HostSweep(wl, Te, lo, table_dev, row_bytes)
        for _ in range(2):
            hs.step()
        barrier()
        start.record()
        for _ in range(args.steps):
            hs.step()
        end.record()
        barrier()
        ms_e2e = max_over_ranks([start.elapsed_time(end)])[0] / args.steps
        launches_e2e = ops.launch_count() - l0
        barrier()
        ms_copy = max_over_ranks([hs.copy_only_ms(max(3, args.steps // 2))])[0]
        e2e = {"value": Te * world / (ms_e2e * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": hs.h2d * world,
               "d2h_bytes_per_step": hs.d2h * world, "rows_per_step": Te * world, "ms_per_step": ms_e2e,
               "gbs_over_pcie": (hs.h2d + hs.d2h) * world / (ms_e2e * 1e-3) / 1e9,
               "copy_only_ms": ms_copy, "copy_only_rows_per_s": Te * world / (ms_copy * 1e-3),
               "frac_of_copy_only": ms_copy / ms_e2e,
               "what": "one b200_host_layer_sweep call per step: every input row copied from page-locked host memory and "
                       "every result row copied back inside the timed region (weights and the table resident on the "
                       "device; the residual stream stays on the device between the ops); copy_only = the same bytes as "
                       "plain copies in both directions at once, max over ranks"}
        hs.host.close()
        del hs
    del sw
    torch.cuda.empty_cache()

    # ---- the other workloads: per-kernel tables, every launch on cold inputs
    others = {}
    if not args.no_other_configs:
        flush = torch.zeros(96 << 20, device=device, dtype=torch.int32)   # 384 MB, rewritten before every launch
        for name in sorted(WORKLOADS):
            if name == args.config:
                continue
            w2 = WORKLOADS[name]
            lo2, T2, T2_total = rank_rows(w2["T"])
            if T2 <= 0:
                continue
            s2 = Sweep(w2, T2, lo2, device)
            for _ in range(3):
                s2.step()
            l0 = ops.launch_count()
            _, pk = time_sweeps(s2, 5, 4, flush=flush)
            launches += ops.launch_count() - l0
            # What a launch of this length can reach at all: a plain device copy (torch's copy kernel) of each kernel's
            # algorithmic bytes, half read and half written, timed the same way (one launch between two events, L2
            # flushed before it). Launch ramp and tail weigh the same on it.
            copies = []
            for (_, _, nbytes, _, _) in s2.kernels:
                a_ = torch.empty(max(nbytes // 2, 16), device=device, dtype=torch.uint8)
                b_ = torch.empty_like(a_)
                ts = []
                for i in range(8):
                    flush.add_(1)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    b_.copy_(a_)
                    e1.record()
                    e1.synchronize()
                    if i >= 3:
                        ts.append(e0.elapsed_time(e1))
                copies.append(sum(ts) / len(ts))
                del a_, b_
            copies = max_over_ranks(copies)
            # the whole sweep back to back (warm L2, no events between the launches), as CUDA-graph replays
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                s2.step()
                with torch.cuda.graph(g, stream=side):
                    s2.step()
            torch.cuda.current_stream().wait_stream(side)
            n_rep = 50
            for _ in range(3):
                g.replay()
            barrier()
            start.record()
            for _ in range(n_rep):
                g.replay()
            end.record()
            barrier()
            launches += len(s2.kernels) * n_rep
            sweep_ms = max_over_ranks([start.elapsed_time(end)])[0] / n_rep
            others[name] = {"workload": w2["name"], "dtype": w2["dtype"], "token_rows_total": T2_total, "token_rows_per_gpu": T2,
                            "sweep_ms_graph_replay": sweep_ms, "rows_per_s": T2_total / (sweep_ms * 1e-3),
                            "kernels": kernel_table(s2, pk, world, peak, time_sweeps.median, time_sweeps.best),
                            "timing": "per kernel: CUDA events around single launches, L2 flushed (384 MB rewritten) "
                                      "before each; sweep: 50 CUDA-graph replays back to back; same_bytes_copy_ms: a plain "
                                      "device copy of the kernel's algorithmic bytes timed the same way"}
            for krow, cms in zip(others[name]["kernels"], copies):
                krow["same_bytes_copy_ms"] = cms
                krow["frac_of_same_bytes_copy"] = cms / krow["ms"]
            del s2, g
            torch.cuda.empty_cache()
        del flush

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        torch.cuda.empty_cache()
        rows = args.cpu_rows or cpu_sample_rows(wl, 4.0)
        cs, dt = time_cpu(wl, rows, 3, 1)
        cpu = {"value": rows / dt, "unit": "rows/s", "cores": cs.threads, "kind": cs.kind,
               "sample": f"{rows} token rows of the same sweep per step, 3 steps, fp32 (the reference's CPU precision), "
                         f"{cs.threads} host threads"}
        # one thread, which is how the reference runs its embedding decode (src/qwen_model.cpp:980): a smaller sample
        rows1 = max(256, rows // 16)
        _, dt1 = time_cpu(wl, rows1, 2, 1, threads=1)
        cpu["single_thread"] = {"value": rows1 / dt1, "unit": "rows/s", "cores": 1, "sample": f"{rows1} token rows, 2 steps"}

    if rank == 0:
        line = {
            "metric": "layer-op sweep throughput (token rows/s)", "value": T_total * reps / (ms_step * 1e-3), "unit": "rows/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": wl["dtype"],
            "data": "synthetic",
            "config": {"workload": f"{args.config}: {wl['name']}", "token_rows_total": T_total, "token_rows_per_gpu": T,
                       "sweeps_per_step": reps, "ms_per_sweep": ms_step / reps,
                       "hidden": wl["E"], "ffn": wl["FF"], "heads": [wl["n_q"], wl["n_kv"], wl["D"]],
                       "parallelism": f"row-sharded x{world}, no collective on the data path (NCCL carries only the "
                                      f"harness's barrier and max-reduce)",
                       "cache": cache_note},
            "step_timed_as": "cuda graph replay" if graph_ms is not None else "individual launches",
            "kernels": kernels, "roofline": roof, "configs": others, "e2e": e2e, "cpu_baseline": cpu, "clocks": clk,
            "gpu_launches": launches, "gpu_launches_e2e": launches_e2e,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def sw_bytes(wl):
    return 2 if wl["dtype"] == "bf16" else 4


if __name__ == "__main__":
    main()
