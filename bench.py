#!/usr/bin/env python
"""Benchmark of the fused layer-op path: one step = one pass of the layer-op sweep over one batch of synthetic rows
(embedding gather -> RMSNorm -> q/k norm + RoPE -> residual add + RMSNorm -> SwiGLU -> residual add + RMSNorm), in the
order a layer of the reference's forward pass issues them (src/qwen_model.cpp:980-990, 941-957).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c5|c4|c3|c1] [--impl reference]

For N > 1 launch one process per GPU with torch.distributed.run; rows are sharded by token, no collective touches
the data path (torch.distributed only carries the barrier and the max over ranks of the device-timed duration).
Prints ONE JSON line on rank 0:
  value       token rows per second through the whole sweep, inputs resident in HBM, all ranks together
  kernels     per kernel: rows/s, algorithmic GB/s, fraction of the measured HBM copy peak and of the nominal 8 TB/s
  roofline    the dominant kernel (SwiGLU) against the measured HBM peak
  e2e         the same sweep through the host-buffer C-ABI calls, host<->device copies inside the timed region
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

# Workloads (BASELINE.json configs): row counts and widths. c5 is the headline multi-GPU configuration.
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
        K.append(("qk_norm_rope", lambda: ops.gpu_qk_norm_rope(self.q, self.k, self.qn, self.kn, self.q_out, self.k_out, nq, nkv, D,
                                                               wl["n_rot"], 0, self.positions, self.pos0, T, wl["theta"], eps, gated, 1),
                  T * ((nq * qs if not gated else nq * D) + nkv * D + (nq + nkv) * D) * s, T * (nq + nkv), "head rows"))
        K.append(("add_rmsnorm_ffn", lambda: ops.gpu_add_rmsnorm(self.x, self.proj1, self.x_alt, self.w2, self.xn, E, T, eps),
                  T * 4 * E * s + 4 * E, T, "token rows"))
        K.append(("swiglu", lambda: ops.gpu_swiglu(self.g, self.u, self.act, T * FF), T * 3 * FF * s, T, "token rows"))
        K.append(("add_rmsnorm_next", lambda: ops.gpu_add_rmsnorm(self.x_alt, self.proj2, self.x, self.w1, self.xn, E, T, eps),
                  T * 4 * E * s + 4 * E, T, "token rows"))
        self.dominant = "swiglu"

    def step(self, events=None):
        for i, (_, fn, _, _, _) in enumerate(self.kernels):
            if events is not None:
                events[i][0].record()
            fn()
            if events is not None:
                events[i][1].record()


# ------------------------------------------------------------------------------------------------ host-buffer e2e

class HostSweep:
    """The same sweep through the host-buffer C-ABI calls: every row input starts in page-locked host memory and every
    row output ends there, each step."""

    def __init__(self, wl, T, row0, table_dev, row_bytes):
        import torch
        import rocm_hip_b200 as ops
        self.wl, self.T, self.ops = wl, T, ops
        dt = torch.bfloat16 if wl["dtype"] == "bf16" else torch.float32
        s = 2 if wl["dtype"] == "bf16" else 4
        E, FF = wl["E"], wl["FF"]
        g = torch.Generator().manual_seed(4242 + row0)
        pin = lambda *shape, dtype=dt: torch.empty(*shape, dtype=dtype).pin_memory()
        rnd = lambda *shape: pin(*shape).copy_(torch.randn(*shape, generator=g).to(dt))
        self.host = ops.HostRows(slot_bytes=48 << 20, n_slots=4)
        self.w = (1 + 0.1 * torch.randn(E, generator=g)).float()
        self.h2d = self.d2h = 0
        self.calls = []
        H = self.host
        if wl.get("moe"):
            rows = T * 8
            x, xn = rnd(T, E), pin(T, E)
            gg, uu, act = rnd(rows, 512), rnd(rows, 512), pin(rows, 512)
            self.calls.append(lambda: H.add_rmsnorm(x, None, None, self.w, xn, E, T, wl["eps"]))
            self.calls.append(lambda: H.swiglu(gg, uu, act, rows, 512))
            self.h2d = T * E * s + 2 * rows * 512 * s
            self.d2h = T * E * s + rows * 512 * s
            self.keep = (x, xn, gg, uu, act)
            return
        nq, nkv, D = wl["n_q"], wl["n_kv"], wl["D"]
        gated = wl.get("gated", 0)
        qs = 2 * D if gated else D
        ids = pin(T, dtype=torch.int32).copy_(torch.randint(0, wl["vocab"], (T,), generator=g, dtype=torch.int32))
        x, x_alt, xn = pin(T, E), pin(T, E), pin(T, E)
        q, k = rnd(T, nq * qs), rnd(T, nkv * D)
        qo, ko = pin(T, nq * D), pin(T, nkv * D)
        qn = (1 + 0.1 * torch.randn(D, generator=g)).float()
        kn = (1 + 0.1 * torch.randn(D, generator=g)).float()
        p1, p2 = rnd(T, E), rnd(T, E)
        gg, uu, act = rnd(T, FF), rnd(T, FF), pin(T, FF)
        eps = wl["eps"]
        C = self.calls
        C.append(lambda: H.embed_rows(wl["qtype"], table_dev, row_bytes, wl["vocab"], ids, x, E, T))
        C.append(lambda: H.add_rmsnorm(x, None, None, self.w, xn, E, T, eps))
        C.append(lambda: H.qk_norm_rope(q, k, qn, kn, qo, ko, nq, nkv, D, wl["n_rot"], 0, None, row0, T, wl["theta"], eps, gated, 1))
        C.append(lambda: H.add_rmsnorm(x, p1, x_alt, self.w, xn, E, T, eps))
        C.append(lambda: H.swiglu(gg, uu, act, T, FF))
        C.append(lambda: H.add_rmsnorm(x_alt, p2, x, self.w, xn, E, T, eps))
        self.h2d = T * (4 + E * s + (nq * qs + nkv * D) * s + 2 * E * s + 2 * FF * s + 2 * E * s)
        self.d2h = T * (E * s + E * s + (nq + nkv) * D * s + 2 * E * s + FF * s + 2 * E * s)
        self.keep = (ids, x, x_alt, xn, q, k, qo, ko, p1, p2, gg, uu, act, qn, kn)

    def step(self):
        for c in self.calls:
            c()


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


def main():
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="total token rows (default: the configuration's)")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: the configuration's rows are sharded over the GPUs; weak: every GPU gets all of them")
    ap.add_argument("--e2e-rows", type=int, default=16384, help="token rows per rank of the host-buffer measurement")
    ap.add_argument("--cpu-rows", type=int, default=0, help="token rows of the CPU sample (default: calibrated)")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="time the step as CUDA-graph replays (auto: when a step is shorter than 1 ms)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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
        dist.init_process_group("nccl", device_id=device)
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

    T_total = args.tokens or wl["T"]
    if args.scaling == "strong":
        lo, hi = shard(T_total, rank, world)
    else:
        lo, hi = rank * T_total, (rank + 1) * T_total
        T_total = T_total * world
    T = hi - lo
    sw = Sweep(wl, T, lo, device)
    nk = len(sw.kernels)
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nk)]
          for _ in range(args.steps)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    clocks = ClockSampler(local)
    clocks.start()
    for _ in range(max(args.warmup, 3)):
        sw.step()
    launches0 = ops.launch_count()
    barrier()
    clocks.mark_begin()
    start.record()
    for i in range(args.steps):
        sw.step(ev[i])
    end.record()
    barrier()
    clocks.mark_end()
    clk = clocks.stop()
    launches = ops.launch_count() - launches0
    ms_total = start.elapsed_time(end)
    per_kernel_ms = [sum(ev[i][j][0].elapsed_time(ev[i][j][1]) for i in range(args.steps)) / args.steps for j in range(nk)]
    red = max_over_ranks([ms_total] + per_kernel_ms)
    ms_step = red[0] / args.steps
    per_kernel_ms = red[1:]
    # Latency-bound workloads (a step of a few microseconds of device work per kernel): the six launches of a step are
    # captured once in a CUDA graph and the step is timed as graph replays, which takes the Python launch overhead out
    # of the number. The per-kernel figures above stay those of the individual launches.
    graph_ms = None
    if args.graph == "on" or (args.graph == "auto" and ms_step < 1.0):
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
        for _ in range(args.steps):
            g.replay()
        end.record()
        barrier()
        launches += nk * args.steps
        graph_ms = max_over_ranks([start.elapsed_time(end)])[0] / args.steps
        ms_step = graph_ms
    if not wl.get("moe"):
        assert int(sw.bad.item()) == 2**31 - 1

    peak, peak_src = measured_peak()
    kernels = []
    roof = None
    for (name, _, nbytes, rows, unit), ms in zip(sw.kernels, per_kernel_ms):
        gbs = nbytes * world / (ms * 1e-3) / 1e9 if args.scaling == "strong" or True else 0
        per_gpu_gbs = nbytes / (ms * 1e-3) / 1e9
        kernels.append({"name": name, "ms": ms, "rows_per_s": rows * world / (ms * 1e-3), "rows": unit,
                        "algorithmic_bytes_per_gpu": nbytes, "gbs_per_gpu": per_gpu_gbs, "gbs_all_gpus": gbs,
                        "frac_of_measured_peak": per_gpu_gbs / peak, "frac_of_8tbs": per_gpu_gbs / NOMINAL_HBM_GBS})
        if name == sw.dominant:
            # DRAM bytes per algorithmic byte of the SwiGLU kernel from one ncu capture at 16,384 tokens
            # (profiles/step_c5_16k_tokens_full.md: dram read + write = 1673.6 MB for 1711.3 MB algorithmic; the last
            # writes of a launch are still in L2 when it ends). Traffic grows in proportion to the rows.
            traffic = 0.978 * nbytes
            roof = {"kernel": name, "bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s",
                    "frac": per_gpu_gbs / peak, "traffic": traffic, "peak_source": f"of {peak_src}",
                    "algorithmic_bytes_per_launch": nbytes, "ms_per_launch": ms}

    # ---- end to end through the host-buffer calls
    e2e = None
    if not args.no_e2e:
        Te = min(args.e2e_rows, T)
        hs = HostSweep(wl, Te, lo, getattr(sw, "table", None), getattr(sw, "row_bytes", 0))
        for _ in range(2):
            hs.step()
        barrier()
        start.record()
        for _ in range(args.steps):
            hs.step()
        end.record()
        barrier()
        ms_e2e = max_over_ranks([start.elapsed_time(end)])[0] / args.steps
        e2e = {"value": Te * world / (ms_e2e * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": hs.h2d * world,
               "d2h_bytes_per_step": hs.d2h * world, "rows_per_step": Te * world, "ms_per_step": ms_e2e,
               "what": "every row input copied from page-locked host memory and every row output copied back, each "
                       "step, through the b200_host_* calls (weights resident on the device)"}
        launches_e2e = ops.launch_count() - launches0 - launches
        hs.host.close()
        del hs
    else:
        launches_e2e = 0

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        del sw
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
            "metric": "layer-op sweep throughput (token rows/s)", "value": T_total / (ms_step * 1e-3), "unit": "rows/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": wl["dtype"],
            "data": "synthetic",
            "config": {"workload": f"{args.config}: {wl['name']}", "token_rows_total": T_total, "token_rows_per_gpu": T,
                       "hidden": wl["E"], "ffn": wl["FF"], "heads": [wl["n_q"], wl["n_kv"], wl["D"]],
                       "parallelism": f"row-sharded x{world}, no collective",
                       "cache": "every tensor of a step is larger than L2 (126 MB); no flush needed" if T * wl["E"] * sw_bytes(wl) > 126e6
                       else "working set near L2 size: latency-bound configuration"},
            "step_timed_as": "cuda graph replay" if graph_ms is not None else "individual launches",
            "kernels": kernels, "roofline": roof, "e2e": e2e, "cpu_baseline": cpu, "clocks": clk,
            "gpu_launches": launches, "gpu_launches_e2e": launches_e2e,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def sw_bytes(wl):
    return 2 if wl["dtype"] == "bf16" else 4


if __name__ == "__main__":
    main()
