#!/usr/bin/env python
"""Benchmark of the batched prediction path on the fixed batch of the scale sweep.

One JSON line on stdout (rank 0).  A step is one pass over the whole batch: 67,108,872
(kernel x destination) pairs of wave scaling (11,184,812 kernels to six device rows) plus
16,777,216 MLP queries (4,194,304 for each of the conv2d, linear, bmm and lstm predictors).
Under torchrun (one rank per GPU) the batch is sharded: every rank takes a contiguous range of
kernels and of each predictor's queries, and each step ends its two phases with the all-reduce
of the per-destination totals ([6] for the pairs, [4 x 6] for the queries) inside the timed
region: by default inside the final stage of the reductions, through mailboxes in the peer GPUs'
memory (`--totals nccl`: NCCL all-reduces).  The same command on one GPU runs the whole batch
(strong scaling).

The headline `value` is wave-scaled pairs per second over the wave-scaling phases of the timed
steps; the `mlp` object carries predictions per second over the MLP phases.  Both are measured
three ways: on the device with inputs resident in HBM (`value`), end to end from pinned host
buffers through the host pipelines of the package (`e2e`), and on the host cores with the CPU
oracle (`cpu_baseline`).  Kernel-only timings of the single-GPU configurations (1,048,576
kernels; conv2d predictor on 262,144 queries; linear predictor in split precision on 65,536
queries), the mixed iteration trace and the multi-GPU result check ride along as sub-entries.
`--impl reference` times only the CPU implementation.  `--case NAME` runs one sub-entry alone
(a small command for profilers).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

# torchrun pins OMP_NUM_THREADS to 1; the CPU baseline is meant to use every host core
os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

import numpy as np  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WAVE_D = 6
WAVE_BYTES_PER_PAIR = 25.0 / WAVE_D + 9.0   # 20 B read + 5 B written per kernel, 9 B per pair
CONFIG2_K = 1 << 20
CONFIG2_SETS = 4                            # rotating buffer sets: 4 x 83 MB > 126 MB of L2
CONFIG3_Q = 262144
CONFIG1_Q = 65536
L2_FLUSH_BYTES = 256 << 20
E2E_CHUNK_K = 1 << 20
E2E_CHUNK_Q = 262144


def mlp_flops_per_query(n_op_features):
    return 2 * ((n_op_features + 4) * 1024 + 8 * 1024 * 1024 + 1024)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the bench runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.samples = []
        self.proc = None
        self.gpu_index = gpu_index
        self.marks = {}

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._pump, daemon=True).start()

    def _pump(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def mark(self, name):
        self.marks[name] = time.time()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self):
        rows = []
        t0, t1 = self.marks.get("timed_start", 0), self.marks.get("timed_end", float("inf"))
        for ts, line in self.samples:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                rows.append((ts, float(parts[0]), float(parts[1]), parts[3:7]))
            except ValueError:
                continue
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        inside = [r for r in rows if t0 <= r[0] <= t1] or rows
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in inside for n, v in zip(names, r[3]) if v.lower().startswith("active")})
        return {"sm_mhz": float(np.median([r[1] for r in inside])), "sm_max_mhz": inside[0][2],
                "reasons": reasons, "samples": len(inside)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), \
        int(os.environ.get("WORLD_SIZE", 1))


SWEEP_WORKLOAD = ("config 5: scale sweep, a fixed batch of 67,108,872 wave-scaling pairs (11,184,812 synthetic "
                  "kernels from a V100-class origin to 6 device rows) plus 16,777,216 MLP queries (4,194,304 each "
                  "for the conv2d, linear, bmm and lstm predictors), sharded over the GPUs")


# ---------------------------------------------------------------------------
# CPU legs (the oracle; the only places the benchmark executes oracle/)
# ---------------------------------------------------------------------------
def cpu_wave(target_s=8.0, repeats=1):
    """Times the C oracle (OpenMP, all host cores) on a sample sized for about
    `target_s` seconds per pass; `repeats` passes over the same sample."""
    from habitat_b200 import device_table, workloads
    from oracle import wave as owave
    devs = device_table.load_device_file()
    specs = [devs[n].spec_tuple() for n in workloads.BENCH_DEVICES]
    k = workloads.sweep_kernels(0, 1 << 17)
    owave.wave_scale_batch(specs, 0, list(range(WAVE_D)), k, want_limits=False)
    t = time.perf_counter()
    r = owave.wave_scale_batch(specs, 0, list(range(WAVE_D)), k, want_limits=False)
    rate = (1 << 17) * WAVE_D / (time.perf_counter() - t)
    n = int(min(max(rate * target_s / WAVE_D, 1 << 17), workloads.SWEEP_KERNELS))
    k = workloads.sweep_kernels(0, n)
    # when the whole batch takes less than the target, a timed unit is several passes over it
    inner = max(1, int(round(target_s / max(n * WAVE_D / rate, 1e-3)))) if n == workloads.SWEEP_KERNELS else 1
    times = []
    for _ in range(repeats):
        t = time.perf_counter()
        for _ in range(inner):
            r = owave.wave_scale_batch(specs, 0, list(range(WAVE_D)), k, want_limits=False)
        times.append(time.perf_counter() - t)
    dt = float(np.mean(times))
    return {"value": inner * n * WAVE_D / dt, "unit": "pairs/s", "cores": int(r["threads"]), "kind": "port",
            "sample": "%d pass(es) over the first %d kernels of the batch x %d devices, C oracle under OpenMP, "
                      "%.1f s" % (inner, n, WAVE_D, dt), "seconds": times, "pairs": inner * n * WAVE_D}


def cpu_mlp(target_s=10.0, repeats=1):
    """Times the numpy/BLAS float32 forward of the four predictors on the first queries of
    each predictor's batch, about `target_s` seconds per pass in all."""
    from habitat_b200 import workloads
    from oracle import mlp as omlp
    ops = workloads.SWEEP_OPS
    w = {op: workloads.torch_init_mlp_weights(op) for op in ops}
    stats = {op: workloads.sweep_mu_sigma(op) for op in ops}
    f, d = workloads.sweep_queries("linear", 0, 4096)
    t = time.perf_counter()
    omlp.predict(w["linear"], f, d, workloads.BENCH_DEVICE_FEATURES, *stats["linear"])
    rate = 4096 / (time.perf_counter() - t)
    n = int(min(max(rate * target_s / len(ops), 2048), 1 << 18))
    data = {op: workloads.sweep_queries(op, 0, n) for op in ops}
    times = []
    for _ in range(repeats):
        t = time.perf_counter()
        for op in ops:
            omlp.predict(w[op], data[op][0], data[op][1], workloads.BENCH_DEVICE_FEATURES, *stats[op])
        times.append(time.perf_counter() - t)
    dt = float(np.mean(times))
    return {"value": n * len(ops) / dt, "unit": "predictions/s", "cores": os.cpu_count(), "kind": "port",
            "sample": "the first %d queries of each of the four predictors, float32 numpy/BLAS forward of the "
                      "same weights, %.1f s per pass" % (n, dt), "seconds": times, "queries": n * len(ops)}


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    steps = max(1, args.steps)
    per = args.cpu_seconds if args.cpu_seconds > 0 else max(0.5, min(6.0, 60.0 / (steps + args.warmup)))
    wave = cpu_wave(target_s=per, repeats=steps + args.warmup)
    timed = wave.pop("seconds")[args.warmup:]
    wave_s = float(np.sum(timed))
    wave["value"] = wave.pop("pairs") * len(timed) / wave_s
    mlp = cpu_mlp(target_s=per, repeats=steps + args.warmup)
    mtimed = mlp.pop("seconds")[args.warmup:]
    mlp_s = float(np.sum(mtimed))
    mlp["value"] = mlp.pop("queries") * len(mtimed) / mlp_s
    line = {
        "impl": "reference", "metric": "wave_scaled_kernel_pairs_per_sec", "value": wave["value"],
        "unit": "pairs/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * (wave_s + mlp_s) / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "i32+f64", "data": "synthetic",
        "config": {"workload": SWEEP_WORKLOAD,
                   "sample": "each step a bounded sample of that batch (its first kernels and queries) on the host "
                             "cores: the C oracle under OpenMP and the numpy/BLAS forward of the four predictors"},
        "cpu_baseline": wave,
        "e2e": {"value": wave["value"], "unit": "pairs/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "mlp": {"metric": "mlp_predictions_per_sec", "value": mlp["value"], "unit": "predictions/s",
                "cpu_baseline": mlp,
                "e2e": {"value": mlp["value"], "unit": "predictions/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class Ctx:
    """What every part of the GPU arm needs: ranks, devices, the stream, helpers."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        from habitat_b200 import device_table, workloads
        from habitat_b200 import distributed as hd
        self.torch, self.dist, self.hd = torch, dist, hd
        self.args = args
        self.rank, self.local_rank, self.world = dist_env()
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            # NCCL prints its version banner on stdout with the first communicator; stdout carries
            # the one JSON line only, so the banner goes to stderr
            sys.stdout.flush()
            saved = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
                warm = torch.zeros(1, device="cuda")
                dist.all_reduce(warm)
                torch.cuda.synchronize()
                hd.host_group()
            finally:
                sys.stdout.flush()
                os.dup2(saved, 1)
                os.close(saved)
        # Totals across ranks: by default exchanged inside the reduction kernels through peer
        # memory (habitat_b200/csrc/peer_exchange.cu), with NCCL all-reduces as the other choice,
        # as the cross-check in the warm-up steps and as the fallback if the set-up fails anywhere.
        self.peer = None
        self.totals_via = "nccl" if self.world > 1 else "none"
        if self.world > 1 and args.totals == "peer":
            ok = 1.0
            try:
                self.peer = hd.PeerTotals()
                self.peer.set_wait(4.0)      # a rank may stall for a moment (host jitter) without failing the run
            except Exception as exc:                       # noqa: BLE001 - any failure means NCCL
                print("peer exchange unavailable on rank %d: %s" % (self.rank, exc), file=sys.stderr)
                ok = 0.0
            flag = torch.tensor([ok], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if float(flag.item()) == 1.0:
                self.totals_via = "peer"
            else:
                self.peer = None
        self.peaks = load_peaks()
        devs = device_table.load_device_file()
        self.bench_devs = [devs[n] for n in workloads.BENCH_DEVICES]
        self.origin = self.bench_devs[0]
        self.stream = torch.cuda.Stream()
        self.launches = 0

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def reduce(self, value, op="max"):
        if self.world == 1:
            return value
        t = self.torch.tensor([value], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.MIN)
        return float(t.item())

    def event(self):
        return self.torch.cuda.Event(enable_timing=True)


def replay_timed(ctx, graph, launches_per_replay, min_ms=50.0):
    """ms per launch of a captured graph: replayed back to back until the timed region is at
    least `min_ms` long."""
    torch = ctx.torch
    graph.replay()
    e0, e1 = ctx.event(), ctx.event()
    e0.record(ctx.stream)
    graph.replay()
    e1.record(ctx.stream)
    torch.cuda.synchronize()
    once = max(e0.elapsed_time(e1), 1e-3)
    n = max(1, int(math.ceil(min_ms / once)))
    e0.record(ctx.stream)
    for _ in range(n):
        graph.replay()
    e1.record(ctx.stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (n * launches_per_replay), n * launches_per_replay


def case_config2_inputs(ctx, mode):
    """Kernel-only timing of configuration 2 with the analyzer's real inputs: the status plane,
    per-destination register counts (MetadataManager), or gamma from raw metrics."""
    torch = ctx.torch
    from habitat_b200 import batched, workloads
    reps = 20
    with torch.cuda.stream(ctx.stream):
        kbs = [batched.KernelBatch.from_numpy(workloads.make_kernels(CONFIG2_K, 1002 + 17 * s))
               for s in range(CONFIG2_SETS)]
        kw = {}
        if mode == "status":
            kw = dict(want_status=True)
        elif mode == "regs":
            regs = workloads.rng(3).integers(-1, 256, size=(WAVE_D, CONFIG2_K)).astype(np.int16)
            kw = dict(dest_regs=torch.from_numpy(regs).cuda())
        elif mode == "metrics":
            m = workloads.make_metrics(CONFIG2_K, 5)
            kw = dict(metrics=batched.KernelMetricsBatch(*[torch.from_numpy(m[n]).cuda() for n in (
                "flop_efficiency_pct", "dram_read_bytes", "dram_write_bytes", "has_metrics")]))
        outs = [batched.wave_scale(kbs[s], ctx.origin, ctx.bench_devs, **kw) for s in range(CONFIG2_SETS)]
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=ctx.stream):
            for i in range(reps):
                batched.wave_scale(kbs[i % CONFIG2_SETS], ctx.origin, ctx.bench_devs, out=outs[i % CONFIG2_SETS], **kw)
        ms, n = replay_timed(ctx, g, reps)
        ctx.launches += n
    return {"workload": "config 2 (1,048,576 kernels x 6 rows per launch) with " +
                        {"status": "the status plane", "regs": "per-destination register counts",
                         "metrics": "gamma from raw metrics"}[mode],
            "kernel": batched.wave_scale_path(), "us_per_launch": ms * 1e3, "launches_timed": n}


def case_config2(ctx, small=True, large=True):
    """Kernel-only and per-step timing of configuration 2 (1,048,576 kernels x 6 rows per launch),
    and of the same kernel on a batch eight times as large."""
    torch = ctx.torch
    from habitat_b200 import batched, workloads
    peaks = ctx.peaks
    reps = 40
    out = {}
    with torch.cuda.stream(ctx.stream):
        if not small:
            return case_config2_large(ctx)
        kbs = [batched.KernelBatch.from_numpy(workloads.make_kernels(CONFIG2_K, 1002 + 17 * s))
               for s in range(CONFIG2_SETS)]
        outs = [batched.wave_scale(kbs[s], ctx.origin, ctx.bench_devs) for s in range(CONFIG2_SETS)]
        totals = torch.zeros((reps, WAVE_D), dtype=torch.float64, device="cuda")
        batched.plane_sum(outs[0].scaled_ns, out=totals[0])
        torch.cuda.synchronize()
        g_kernel, g_step = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_kernel, stream=ctx.stream):
            for i in range(reps):
                batched.wave_scale(kbs[i % CONFIG2_SETS], ctx.origin, ctx.bench_devs, out=outs[i % CONFIG2_SETS])
        # a step = the kernel, whose blocks add up their own results, plus the final stage of the
        # per-destination totals
        parts = [batched.WavePartials(CONFIG2_K, WAVE_D) for _ in range(CONFIG2_SETS)]
        with torch.cuda.graph(g_step, stream=ctx.stream):
            for i in range(reps):
                s = i % CONFIG2_SETS
                batched.wave_scale(kbs[s], ctx.origin, ctx.bench_devs, out=outs[s], partials=parts[s])
                parts[s].totals(out=totals[i])
        kern_ms, n_k = replay_timed(ctx, g_kernel, reps)
        step_ms, n_s = replay_timed(ctx, g_step, reps)
        pairs = CONFIG2_K * WAVE_D
        gbs = pairs * WAVE_BYTES_PER_PAIR / (kern_ms * 1e-3) / 1e9
        out = {"workload": "config 2: 1,048,576 kernels x 6 device rows per launch, %d rotating buffer sets "
                           "(%.0f MB) so that no launch finds its data in L2, graph replay"
                           % (CONFIG2_SETS, CONFIG2_SETS * pairs * WAVE_BYTES_PER_PAIR / 1e6),
               "kernel": batched.wave_scale_path(), "us_per_launch": kern_ms * 1e3, "launches_timed": n_k,
               "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
               "us_per_step": step_ms * 1e3, "steps_timed": n_s,
               "pairs_per_s_step": pairs / (step_ms * 1e-3)}
        ctx.launches += n_k + 2 * n_s
        del kbs, outs, g_kernel, g_step
        if large:
            out["large_batch"] = case_config2_large(ctx)
    return out


def case_config2_large(ctx):
    """The table kernel on 8,388,608 kernels per launch (two buffer sets, 1.3 GB)."""
    torch = ctx.torch
    from habitat_b200 import batched, workloads
    with torch.cuda.stream(ctx.stream):
        big_k = 8 * CONFIG2_K
        big = [batched.KernelBatch.from_numpy(workloads.make_kernels(big_k, 7001 + s)) for s in range(2)]
        big_out = [batched.wave_scale(big[s], ctx.origin, ctx.bench_devs) for s in range(2)]
        torch.cuda.synchronize()
        g_big = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_big, stream=ctx.stream):
            for i in range(6):
                batched.wave_scale(big[i % 2], ctx.origin, ctx.bench_devs, out=big_out[i % 2])
        big_ms, n_b = replay_timed(ctx, g_big, 6)
        big_gbs = big_k * WAVE_D * WAVE_BYTES_PER_PAIR / (big_ms * 1e-3) / 1e9
        ctx.launches += n_b
        return {"kernels": big_k, "us_per_launch": big_ms * 1e3, "achieved": big_gbs,
                "frac": big_gbs / ctx.peaks["hbm_gbs"], "launches_timed": n_b}


def case_config2_totals(ctx):
    """Per-destination totals of the predicted times, two ways, per launch size: the table kernel
    followed by the two-stage plane sum over its results, and the table kernel whose blocks add up
    their own results followed by the final stage alone.  Graph replay, four rotating buffer sets."""
    torch = ctx.torch
    from habitat_b200 import batched, workloads
    rows = []
    with torch.cuda.stream(ctx.stream):
        for K in (CONFIG2_K, workloads.SWEEP_KERNELS // 16 * 2, workloads.SWEEP_KERNELS):
            sets, reps = 4, 20
            kbs = [batched.KernelBatch.from_numpy(workloads.make_kernels(K, 1002 + 17 * s)) for s in range(sets)]
            parts = [batched.WavePartials(K, WAVE_D) for _ in range(sets)]
            outs = [batched.wave_scale(kbs[s], ctx.origin, ctx.bench_devs, partials=parts[s]) for s in range(sets)]
            totals = torch.zeros((reps, WAVE_D), dtype=torch.float64, device="cuda")
            parts[0].totals(out=totals[0])
            batched.plane_sum(outs[0].scaled_ns, out=totals[1])
            torch.cuda.synchronize()
            row = {"kernels": K, "first_stage_sums_per_destination": parts[0].per_plane}
            for name, fused, final in (("kernel", False, False), ("kernel_then_plane_sum", False, True),
                                       ("kernel_with_block_sums", True, False),
                                       ("kernel_with_block_sums_then_final_stage", True, True)):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=ctx.stream):
                    for i in range(reps):
                        q = i % sets
                        batched.wave_scale(kbs[q], ctx.origin, ctx.bench_devs, out=outs[q],
                                           partials=parts[q] if fused else None)
                        if final and fused:
                            parts[q].totals(out=totals[i])
                        elif final:
                            batched.plane_sum(outs[q].scaled_ns, out=totals[i])
                ms, n = replay_timed(ctx, g, reps)
                row["us_" + name] = ms * 1e3
                ctx.launches += n * (1 + (2 if final and not fused else int(final)))
                del g
            rows.append(row)
            del kbs, parts, outs
    return {"workload": "per-destination totals of the predicted times, 6 device rows", "launch_sizes": rows}


def case_sweep_kernel(ctx):
    """The default run's own wave-scaling launch alone: the table kernel with block sums on the
    sweep's 11,184,812 kernels, two buffer sets (1.7 GB, so no launch finds its data in L2), two
    warm-up and six timed launches.  A small command for profilers."""
    torch = ctx.torch
    from habitat_b200 import batched, workloads
    K = workloads.SWEEP_KERNELS
    with torch.cuda.stream(ctx.stream):
        kbs = [batched.KernelBatch.from_numpy(workloads.sweep_kernels(0, K)),
               batched.KernelBatch.from_numpy(workloads.make_kernels(K, 4242))]
        parts = [batched.WavePartials(K, WAVE_D) for _ in range(2)]
        outs = [batched.wave_scale(kbs[q], ctx.origin, ctx.bench_devs, partials=parts[q]) for q in range(2)]
        torch.cuda.synchronize()
        e0, e1 = ctx.event(), ctx.event()
        e0.record(ctx.stream)
        for i in range(6):
            batched.wave_scale(kbs[i % 2], ctx.origin, ctx.bench_devs, out=outs[i % 2], partials=parts[i % 2])
        e1.record(ctx.stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 6
        ctx.launches += 8
    gbs = K * WAVE_D * WAVE_BYTES_PER_PAIR / (us * 1e-6) / 1e9
    return {"workload": "the sweep's wave-scaling launch alone (11,184,812 kernels x 6 device rows, block sums)",
            "kernel": batched.wave_scale_path(), "kernels": K, "first_stage_sums_per_destination": parts[0].per_plane,
            "us_per_launch": us, "achieved": gbs, "peak": ctx.peaks["hbm_gbs"], "unit": "GB/s",
            "frac": gbs / ctx.peaks["hbm_gbs"], "launches_timed": 6}


def case_config3(ctx):
    """Kernel-only timing of configuration 3: conv2d predictor, 262,144 queries, bf16."""
    torch = ctx.torch
    from habitat_b200 import batched, workloads
    op = "conv2d"
    with torch.cuda.stream(ctx.stream):
        w = workloads.torch_init_mlp_weights(op)
        feats, dev = workloads.make_queries(op, CONFIG3_Q, 1003)
        mu, sigma = workloads.batch_mu_sigma(feats, dev)
        h = batched.MLPHandle(feats.shape[1], mu=mu, sigma=sigma,
                              device_features=workloads.BENCH_DEVICE_FEATURES, **w)
        d_f, d_r = torch.from_numpy(feats).cuda(), torch.from_numpy(dev).cuda()
        d_o = torch.empty((CONFIG3_Q,), dtype=torch.float32, device="cuda")
        for _ in range(3):
            h.predict(d_f, d_r, out=d_o)
        h.check_status()
        n = 16
        e0, e1 = ctx.event(), ctx.event()
        e0.record(ctx.stream)
        for _ in range(n):
            h.predict(d_f, d_r, out=d_o)
        e1.record(ctx.stream)
        torch.cuda.synchronize()
        h.check_status()
        ms = e0.elapsed_time(e1) / n
        pc = h.phase_cycles()
        h.close()
    ctx.launches += n
    flops = mlp_flops_per_query(8)
    tf = CONFIG3_Q * flops / (ms * 1e-3) / 1e12
    return {"workload": "config 3: conv2d predictor (8 x 1024 hidden), 262,144 queries per launch, bf16 tensor "
                        "cores, fp32 accumulate", "kernel": "mlp_chain_pair_kernel", "ms_per_launch": ms,
            "launches_timed": n, "achieved": tf, "peak": ctx.peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": tf / ctx.peaks["bf16_tflops"], "frac_of_sustained": tf / ctx.peaks["bf16_tflops_sustained"],
            "sm_mhz_in_kernel": 1e3 * pc["mma_total_cycles"] / pc["mma_total_ns"] if pc["mma_total_ns"] > 0 else None,
            "predictions_per_s": CONFIG3_Q / (ms * 1e-3)}


def case_config1(ctx):
    """Configuration 1: linear predictor, 65,536 queries, split precision (the 1e-4 configuration):
    kernel-only time, end to end through the host pipeline, and the CPU forward beside it."""
    torch = ctx.torch
    from habitat_b200 import batched, hostio, workloads
    Q = CONFIG1_Q
    with torch.cuda.stream(ctx.stream):
        w1 = workloads.torch_init_mlp_weights("linear")
        f1, r1 = workloads.make_queries("linear", Q, 1001)
        mu1, sigma1 = workloads.batch_mu_sigma(f1, r1)
        h1 = batched.MLPHandle(f1.shape[1], mu=mu1, sigma=sigma1, precision="bf16x3",
                               device_features=workloads.BENCH_DEVICE_FEATURES, **w1)
        d_f1, d_r1 = torch.from_numpy(f1).cuda(), torch.from_numpy(r1).cuda()
        d_o1 = torch.empty((Q,), dtype=torch.float32, device="cuda")
        for _ in range(3):
            h1.predict(d_f1, d_r1, out=d_o1)
        h1.check_status()
        n = 12
        c0, c1 = ctx.event(), ctx.event()
        c0.record(ctx.stream)
        for _ in range(n):
            h1.predict(d_f1, d_r1, out=d_o1)
        c1.record(ctx.stream)
        torch.cuda.synchronize()
        h1.check_status()
        ms1 = c0.elapsed_time(c1) / n
    ctx.launches += n
    # end to end: pinned features in, pinned predictions out, three batches in flight
    p_f, p_r = torch.from_numpy(f1).pin_memory(), torch.from_numpy(r1).pin_memory()
    pipe = hostio.MLPPredictHost(f1.shape[1], Q, depth=3)
    for i in range(3):
        pipe.submit(h1, p_f, p_r, i % 3)
    torch.cuda.synchronize()
    e0, e1 = ctx.event(), ctx.event()
    e0.record(pipe.s_up)
    n_e = 9
    for i in range(n_e):
        pipe.submit(h1, p_f, p_r, i % 3)
    e1.record(pipe.s_out)
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / n_e
    ctx.launches += n_e + 3
    h1.check_status()
    h1.close()
    tf = Q * mlp_flops_per_query(4) / (ms1 * 1e-3) / 1e12
    return {"workload": "config 1: linear predictor, 65,536 queries, bf16 hi + lo operands (hi and lo parts of the "
                        "activations side by side along N, hi and lo weight tiles accumulated into the same "
                        "columns), tolerance 1e-4", "ms_per_launch": ms1, "value": Q / (ms1 * 1e-3),
            "unit": "predictions/s", "dtype": "bf16x3", "launches_timed": n,
            "roofline": {"bound": "tensor", "kernel": "mlp_chain_pair_kernel<split>", "achieved": tf,
                         "peak": ctx.peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / ctx.peaks["bf16_tflops"],
                         "note": "algorithmic flops; the mode issues two MMAs per K step on tiles of half as many "
                                 "queries, so a quarter of the bf16 peak is its ceiling", "traffic": None},
            "e2e": {"value": Q / (e2e_ms * 1e-3), "unit": "predictions/s",
                    "h2d_bytes_per_step": int(pipe.h2d_bytes), "d2h_bytes_per_step": int(pipe.d2h_bytes)}}


def host_occupancy_fn(origin):
    """(block, smem, regs) arrays -> occupancy on `origin`, evaluated by the library's host-side
    single-record call (rejection sampling of kernels the origin can run)."""
    import ctypes
    from habitat_b200 import _native, device_table
    lib = _native.load()
    row = device_table.row_of(origin)

    def occ(block, smem, regs):
        out = np.empty(len(block), np.int32)
        o = ctypes.c_int32(0)
        for i in range(len(block)):
            lib.hb_thread_block_occupancy(row, int(block[i]), int(smem[i]), int(regs[i]), ctypes.byref(o), None)
            out[i] = o.value
        return out
    return occ


class Sweep:
    """This rank's shard of the fixed batch, resident on its GPU, and the timed step."""

    def __init__(self, ctx, steps_total, klo=None, khi=None, qlo=None, qhi=None, handles=None):
        torch = ctx.torch
        from habitat_b200 import batched, workloads
        self.ctx = ctx
        self.ops = workloads.SWEEP_OPS
        hd = ctx.hd
        if klo is None:
            # cut on the 256 kernels a block of the table kernel takes: a shard's first-stage sums are
            # then the whole batch's, and the sharded totals differ from one GPU's only by the order of
            # the last float64 additions
            klo, khi = hd.shard_bounds_aligned(workloads.SWEEP_KERNELS, ctx.rank, ctx.world, 256)
            qlo, qhi = hd.shard_bounds_aligned(workloads.SWEEP_QUERIES, ctx.rank, ctx.world, 128)
        self.klo, self.khi, self.qlo, self.qhi = klo, khi, qlo, qhi
        self.host_k = workloads.sweep_kernels(klo, khi)
        self.kb = batched.KernelBatch.from_numpy(self.host_k)
        self.partials = batched.WavePartials(khi - klo, WAVE_D)
        self.out = batched.wave_scale(self.kb, ctx.origin, ctx.bench_devs, partials=self.partials)
        self.weights, self.stats, self.host_q = {}, {}, {}
        self.handles = handles if handles is not None else {}
        self.d_f, self.d_r, self.d_o = {}, {}, {}
        for op in self.ops:
            if op not in self.handles:
                self.weights[op] = workloads.torch_init_mlp_weights(op)
                self.stats[op] = workloads.sweep_mu_sigma(op)
                self.handles[op] = batched.MLPHandle(
                    len(workloads.OP_FEATURES[op]), mu=self.stats[op][0], sigma=self.stats[op][1],
                    device_features=workloads.BENCH_DEVICE_FEATURES, **self.weights[op])
            feats, dev = workloads.sweep_queries(op, qlo, qhi)
            self.host_q[op] = (feats, dev)
            self.d_f[op], self.d_r[op] = torch.from_numpy(feats).cuda(), torch.from_numpy(dev).cuda()
            self.d_o[op] = torch.empty((feats.shape[0],), dtype=torch.float32, device="cuda")
        self.totals = torch.zeros((steps_total, WAVE_D + len(self.ops) * WAVE_D), dtype=torch.float64, device="cuda")
        self.flush = torch.empty((L2_FLUSH_BYTES,), dtype=torch.uint8, device="cuda")
        self.ev = []

    def step(self, i, timed=True, via=None):
        """One pass over the shard: wave-scaling phase (the kernel's blocks add up their own results;
        a final stage turns the block sums into the [6] totals), then the MLP phase; each ends with
        the all-reduce of its totals (via "peer": inside the final stage of the reductions, through
        peer memory; via "nccl": one NCCL all-reduce per phase).  Events bracket the phases and
        the dominant kernels."""
        ctx, torch = self.ctx, self.ctx.torch
        from habitat_b200 import batched
        via = via or ctx.totals_via
        s = ctx.stream
        tot = self.totals[i]
        ev = {k: ctx.event() for k in ("w0", "k1", "w1", "m0", "m1")} if timed else None
        self.flush.zero_()                     # the shard's data of the step before must not sit in L2
        if timed:
            ev["w0"].record(s)
        batched.wave_scale(self.kb, ctx.origin, ctx.bench_devs, out=self.out, partials=self.partials)
        if timed:
            ev["k1"].record(s)
        if via == "peer":
            ctx.peer.partials_sum(self.partials, out=tot[:WAVE_D])
        else:
            self.partials.totals(out=tot[:WAVE_D])
            if via == "nccl":
                ctx.dist.all_reduce(tot[:WAVE_D])
        if timed:
            ev["w1"].record(s)
            ev["m0"].record(s)
        pk = []
        for j, op in enumerate(self.ops):
            a = ctx.event() if timed else None
            b = ctx.event() if timed else None
            if timed:
                a.record(s)
            self.handles[op].predict(self.d_f[op], self.d_r[op], out=self.d_o[op])
            if timed:
                b.record(s)
                pk.append((a, b))
            part = tot[WAVE_D * (1 + j):WAVE_D * (2 + j)]
            if via == "peer":
                ctx.peer.group_sum(self.d_o[op], self.d_r[op], WAVE_D, out=part)
            else:
                batched.group_sum(self.d_o[op], self.d_r[op], WAVE_D, out=part)
        if via == "nccl":
            ctx.dist.all_reduce(tot[WAVE_D:])
        if timed:
            ev["m1"].record(s)
            ev["pk"] = pk
            self.ev.append(ev)
        ctx.launches += 2 + 3 * len(self.ops)

    def phase_ms(self):
        w = sum(e["w0"].elapsed_time(e["w1"]) for e in self.ev)
        k = sum(e["w0"].elapsed_time(e["k1"]) for e in self.ev)
        m = sum(e["m0"].elapsed_time(e["m1"]) for e in self.ev)
        per_op = [sum(e["pk"][j][0].elapsed_time(e["pk"][j][1]) for e in self.ev) for j in range(len(self.ops))]
        return w, k, m, per_op


def sweep_totals_alone(ctx, klo, khi, qlo, qhi, handles):
    """Totals of kernels [klo, khi) and queries [qlo, qhi) computed on this GPU alone, no collective:
    numpy [6 + 4 x 6]."""
    torch = ctx.torch
    from habitat_b200 import batched, workloads
    with torch.cuda.stream(ctx.stream):
        tot = torch.zeros((WAVE_D * 5,), dtype=torch.float64, device="cuda")
        kb = batched.KernelBatch.from_numpy(workloads.sweep_kernels(klo, khi))
        out = batched.wave_scale(kb, ctx.origin, ctx.bench_devs)
        batched.plane_sum(out.scaled_ns, out=tot[:WAVE_D])
        for j, op in enumerate(workloads.SWEEP_OPS):
            feats, dev = workloads.sweep_queries(op, qlo, qhi)
            d_f, d_r = torch.from_numpy(feats).cuda(), torch.from_numpy(dev).cuda()
            d_o = handles[op].predict(d_f, d_r)
            batched.group_sum(d_o, d_r, WAVE_D, out=tot[WAVE_D * (1 + j):WAVE_D * (2 + j)])
        torch.cuda.synchronize()
        for h in handles.values():
            h.check_status()
        ctx.launches += 3 + 3 * len(workloads.SWEEP_OPS)
        return tot.cpu().numpy()


def e2e_sweep(ctx, sw):
    """The shard through the host pipelines: pinned record blocks in, pinned predicted times out
    (wave scaling); pinned features in, pinned predictions out (MLP).  Returns ms per pass of each,
    max over ranks, the bytes moved per pass and the plain copy rates of the pipeline's buffers."""
    torch = ctx.torch
    from habitat_b200 import hostio
    n = sw.khi - sw.klo
    chunks = [(a, min(a + E2E_CHUNK_K, n)) for a in range(0, n, E2E_CHUNK_K)]
    with hostio.numa_local(ctx.local_rank):
        blocks = [hostio.pack_kernels({k: v[a:b] for k, v in sw.host_k.items()}) for a, b in chunks]
    full = [c for c in chunks if c[1] - c[0] == E2E_CHUNK_K]
    depth = 3
    pipe = hostio.WaveScaleHost(ctx.origin, ctx.bench_devs, E2E_CHUNK_K, depth=depth) if full else None
    rest = chunks[-1] if chunks and chunks[-1][1] - chunks[-1][0] != E2E_CHUNK_K else None
    pipe_rest = hostio.WaveScaleHost(ctx.origin, ctx.bench_devs, rest[1] - rest[0], depth=1) if rest else None
    join = torch.cuda.Stream()

    def wave_pass(e_end=None):
        for i in range(len(full)):
            pipe.submit(blocks[i], i % depth)
        if rest:
            pipe_rest.submit(blocks[-1], 0)
        if e_end is not None:
            if full:
                join.wait_event(pipe.downloaded[(len(full) - 1) % depth])
            if rest:
                join.wait_event(pipe_rest.downloaded[0])
            e_end.record(join)
    wave_pass()
    ctx.barrier()
    passes = 3
    e0, e1 = ctx.event(), ctx.event()
    e0.record((pipe or pipe_rest).s_up)
    for p in range(passes):
        wave_pass(e1 if p == passes - 1 else None)
    ctx.barrier()
    wave_ms = ctx.reduce(e0.elapsed_time(e1)) / passes
    ctx.launches += (passes + 1) * len(chunks)
    # plain copies of the pipeline's own buffers, all ranks at once: the PCIe / host-memory ceiling
    copy = {}
    if full:
        c0, c1, c2 = ctx.event(), ctx.event(), ctx.event()
        reps = 6
        ctx.barrier()
        c0.record(ctx.stream)
        with torch.cuda.stream(ctx.stream):
            for _ in range(reps):
                pipe.dev_block[0].copy_(blocks[0], non_blocking=True)
            c1.record(ctx.stream)
            for _ in range(reps):
                pipe.host_out[0]["scaled_ns"].copy_(pipe.dev_out[0].scaled_ns, non_blocking=True)
            c2.record(ctx.stream)
        ctx.barrier()
        copy = {"h2d_gbs_per_rank": ctx.reduce(reps * pipe.h2d_bytes / (c0.elapsed_time(c1) * 1e-3) / 1e9, "min"),
                "d2h_gbs_per_rank": ctx.reduce(reps * pipe.d2h_bytes / (c1.elapsed_time(c2) * 1e-3) / 1e9, "min"),
                "ranks_copying_at_once": ctx.world}
    # the same pass for a caller that only wants the per-destination totals of every chunk back
    # (Trace.run_time_ms per destination): 8 x 6 bytes down per chunk instead of 4 bytes per pair
    t_pipe = hostio.WaveScaleHost(ctx.origin, ctx.bench_devs, E2E_CHUNK_K, depth=depth, results=("totals",)) if full else None
    t_rest = hostio.WaveScaleHost(ctx.origin, ctx.bench_devs, rest[1] - rest[0], depth=1, results=("totals",)) if rest else None

    def totals_pass(e_end=None, gather=None):
        for i in range(len(full)):
            if gather is not None:
                t_pipe.wait(i % depth)
                if i >= depth:
                    gather += t_pipe.host_out[i % depth]["totals"].numpy()
            t_pipe.submit(blocks[i], i % depth)
        if rest:
            t_rest.submit(blocks[-1], 0)
        if gather is not None:
            for i in range(max(0, len(full) - depth), len(full)):
                t_pipe.wait(i % depth)
                gather += t_pipe.host_out[i % depth]["totals"].numpy()
            if rest:
                t_rest.wait(0)
                gather += t_rest.host_out[0]["totals"].numpy()
        if e_end is not None:
            if full:
                join.wait_event(t_pipe.downloaded[(len(full) - 1) % depth])
            if rest:
                join.wait_event(t_rest.downloaded[0])
            e_end.record(join)
    chunk_totals = np.zeros(WAVE_D)
    totals_pass(gather=chunk_totals)
    with torch.cuda.stream(ctx.stream):
        from habitat_b200 import batched
        batched.wave_scale(sw.kb, ctx.origin, ctx.bench_devs, out=sw.out, partials=sw.partials)
        shard_totals = sw.partials.totals().cpu().numpy()
    totals_rel = float(np.max(np.abs(chunk_totals - shard_totals) / np.abs(shard_totals))) if n else 0.0
    ctx.barrier()
    t0, t1 = ctx.event(), ctx.event()
    t0.record((t_pipe or t_rest).s_up)
    for p in range(passes):
        totals_pass(t1 if p == passes - 1 else None)
    ctx.barrier()
    totals_ms = ctx.reduce(t0.elapsed_time(t1)) / passes
    totals_rel = ctx.reduce(totals_rel)
    ctx.launches += (passes + 1) * 2 * len(chunks) + 2
    del pipe, pipe_rest, t_pipe, t_rest, blocks

    nq = sw.qhi - sw.qlo
    qchunks = [(a, min(a + E2E_CHUNK_Q, nq)) for a in range(0, nq, E2E_CHUNK_Q)]
    pipes, pinned = {}, {}
    with hostio.numa_local(ctx.local_rank):
        for op in sw.ops:
            f, r = sw.host_q[op]
            pinned[op] = (torch.from_numpy(f).pin_memory(), torch.from_numpy(r).pin_memory())
            pipes[op] = hostio.MLPPredictHost(f.shape[1], E2E_CHUNK_Q, depth=depth)

    def mlp_pass(e_end=None):
        for op in sw.ops:
            f, r = pinned[op]
            for i, (a, b) in enumerate(qchunks):
                pipes[op].submit(sw.handles[op], f[a:b], r[a:b], i % depth)
        if e_end is not None:
            for op in sw.ops:
                join.wait_event(pipes[op].downloaded[(len(qchunks) - 1) % depth])
            e_end.record(join)
    ctx.barrier()
    m0, m1 = ctx.event(), ctx.event()
    m0.record(pipes[sw.ops[0]].s_up)
    mpasses = 2
    for p in range(mpasses):
        mlp_pass(m1 if p == mpasses - 1 else None)
    ctx.barrier()
    mlp_ms = ctx.reduce(m0.elapsed_time(m1)) / mpasses
    ctx.launches += mpasses * len(sw.ops) * len(qchunks)
    for h in sw.handles.values():
        h.check_status()
    h2d_q = sum(sw.host_q[op][0].nbytes + sw.host_q[op][1].nbytes for op in sw.ops)
    return {"wave_ms": wave_ms, "mlp_ms": mlp_ms, "wave_h2d": n * hostio.RECORD_BYTES, "wave_d2h": n * WAVE_D * 4,
            "mlp_h2d": h2d_q, "mlp_d2h": nq * 4 * len(sw.ops), "copy": copy,
            "totals_ms": totals_ms, "totals_d2h": len(chunks) * WAVE_D * 8, "totals_rel": totals_rel}


def config4(ctx, handles, cpu_leg):
    """The mixed iteration trace (512 iterations x 160 operations): per-iteration totals on the
    device, sharded by iteration with an all-gather of the rows; on rank 0 also the same trace
    through the analyzer surface (Trace.to_devices)."""
    torch = ctx.torch
    from habitat_b200 import batched, iteration, workloads
    I = 512
    occ = host_occupancy_fn(ctx.origin)

    def run(lo, hi, gather, every_rank=True):
        sync = ctx.barrier if every_rank else torch.cuda.synchronize
        kernels, overhead, ops = workloads.make_iterations(lo, hi, occ)
        n_it = hi - lo
        with torch.cuda.stream(ctx.stream):
            kb = batched.KernelBatch.from_numpy(kernels)
            d_over = torch.from_numpy(overhead).cuda()
            koff = torch.from_numpy(np.arange(n_it + 1, dtype=np.int64) * workloads.ITER_KERNELS).cuda()
            special = {}
            for op, (feats, rt) in ops.items():
                off = torch.from_numpy(np.arange(n_it + 1, dtype=np.int64) * workloads.ITER_SPECIAL[op]).cuda()
                special[op] = iteration.SpecialOps(handles[op], torch.from_numpy(feats).cuda(),
                                                   torch.from_numpy(rt).cuda(), off)

            def once():
                totals, _ = iteration.predict_iteration_totals(kb, d_over, koff, special, ctx.origin,
                                                               ctx.bench_devs, 0, list(range(WAVE_D)))
                return ctx.hd.allgather_rows(totals) if gather else totals
            rows = once()
            sync()
            e0, e1 = ctx.event(), ctx.event()
            reps = 5
            e0.record(ctx.stream)
            for _ in range(reps):
                rows = once()
            e1.record(ctx.stream)
            sync()
        return rows.cpu().numpy(), e0.elapsed_time(e1) / reps, (kernels, overhead, ops)

    lo, hi = ctx.hd.shard_bounds(I, ctx.rank, ctx.world)
    rows, ms, data = run(lo, hi, ctx.world > 1)
    ms = ctx.reduce(ms)
    for h in handles.values():
        h.check_status()
    out = {"workload": "config 4: 512 iterations x (53 conv2d + 1 linear + 32 bmm MLP-predicted operations + 74 "
                       "wave-scaled kernels) to 6 device rows, %d iterations per GPU, all-gather of the "
                       "[iterations x 6] totals" % (hi - lo),
           "ms_per_pass": ms, "iterations_per_s": I / (ms * 1e-3), "rows": list(rows.shape)}
    if ctx.rank == 0:
        if ctx.world > 1:
            alone, _, data = run(0, I, False, every_rank=False)
            out["matches_one_gpu"] = bool(np.allclose(rows, alone, rtol=1e-12, atol=0))
        if cpu_leg:
            out.update(config4_cpu_check(ctx, rows, data))
            out["analyzer_surface"] = config4_analyzer(ctx, data, handles)
    return out


def config4_cpu_check(ctx, rows, data):
    """cpu_baseline leg: the first 8 iterations against the float64 oracle (2e-2), and the oracle's
    time for the whole trace's arithmetic on the host cores."""
    from habitat_b200 import workloads
    from oracle import mlp as omlp
    from oracle import wave as owave
    kernels, overhead, ops = data
    n_chk = 8
    specs = [d.spec_tuple() for d in ctx.bench_devs]
    devf = workloads.BENCH_DEVICE_FEATURES
    t0 = time.perf_counter()
    ref = owave.wave_scale_batch(specs, 0, list(range(WAVE_D)), kernels, want_limits=False)
    wave_s = time.perf_counter() - t0
    nk = n_chk * workloads.ITER_KERNELS
    want = np.zeros((n_chk, WAVE_D))
    for d in range(WAVE_D):
        ns = kernels["run_time_ns"][:nk] if d == 0 else ref["scaled_ns"][d][:nk]
        want[:, d] = (overhead[:nk].astype(np.float64) + ns).reshape(n_chk, -1).sum(axis=1) / 1e6
    mlp_s = 0.0
    for op, (feats, rt) in ops.items():
        w = workloads.torch_init_mlp_weights(op)
        mu, sigma = workloads.sweep_mu_sigma(op)
        n = n_chk * workloads.ITER_SPECIAL[op]
        t0 = time.perf_counter()
        p_orig = omlp.predict(w, feats[:n], np.zeros(n, np.uint8), devf, mu, sigma, np.float64)
        for d in range(WAVE_D):
            if d == 0:
                ms = rt[:n].astype(np.float64)
            else:
                p_dest = omlp.predict(w, feats[:n], np.full(n, d, np.uint8), devf, mu, sigma, np.float64)
                ms = np.maximum(rt[:n].astype(np.float64) * p_dest / p_orig, 0)
            want[:, d] += ms.reshape(n_chk, -1).sum(axis=1)
        mlp_s += (time.perf_counter() - t0) * len(feats) / max(n, 1)      # scaled to the whole trace
    err = float((np.abs(rows[:n_chk] - want) / np.abs(want)).max())
    return {"max_rel_err_vs_oracle": err, "within_2e-2": bool(err <= 2e-2),
            "cpu_baseline": {"value": wave_s + mlp_s, "unit": "s per pass", "kind": "port", "cores": os.cpu_count(),
                             "sample": "C oracle over all %d kernels (measured) + float64 numpy forward of the MLP "
                                       "operations (measured on %d iterations, scaled to 512)"
                                       % (len(kernels["num_blocks"]), n_chk)}}


def config4_analyzer(ctx, data, handles):
    """The same trace as Python objects through Trace.to_devices (the analyzer's own surface)."""
    torch = ctx.torch
    from habitat_b200 import workloads
    from habitat_b200.analysis.arguments import Arguments
    from habitat_b200.analysis.kernels import MeasuredKernel
    from habitat_b200.analysis.mlp.mlp import RuntimePredictor
    from habitat_b200.analysis.operation import MeasuredOperation
    from habitat_b200.analysis.predictor import Predictor
    from habitat_b200.analysis.run_time import RunTimeMeasurement
    from habitat_b200.analysis.trace import Trace
    from habitat_b200.habitat_cuda import KernelInstance
    kernels, overhead, ops = data
    origin = ctx.origin
    I = len(overhead) // workloads.ITER_KERNELS
    t0 = time.perf_counter()
    operations = []
    nb, bs, rg, sm, tm = (kernels[k] for k in ("num_blocks", "block_size", "regs_per_thread", "smem_bytes",
                                               "run_time_ns"))
    for it in range(I):
        for j in range(workloads.ITER_KERNELS):
            i = it * workloads.ITER_KERNELS + j
            c = KernelInstance("k%d" % j, int(nb[i]), int(bs[i]), int(sm[i]), 0, int(rg[i]), int(tm[i]))
            run = RunTimeMeasurement((float(tm[i]) + float(overhead[i])) / 1e6, [MeasuredKernel(c, [], origin)], origin)
            operations.append(MeasuredOperation("relu", Arguments((), {}), run, None, origin))
        for op, (feats, rt) in ops.items():
            n = workloads.ITER_SPECIAL[op]
            for j in range(it * n, (it + 1) * n):
                f = [int(v) for v in feats[j]]
                if op == "conv2d":
                    bias, batch, image, cin, cout, ksz, stride, pad = f
                    args = ((batch, cin, image, image), (cout, cin, ksz, ksz), (cout,) if bias else None,
                            (stride, stride), (pad, pad), (1, 1), 1)
                elif op == "linear":
                    bias, batch, fin, fout = f
                    args = ((batch, fin), (fout, fin), (fout,) if bias else None)
                else:
                    batch, left, middle, right = f
                    args = ((batch, left, middle), (batch, middle, right))
                operations.append(MeasuredOperation(op, Arguments(args, {}),
                                                    RunTimeMeasurement(float(rt[j]), [], origin), None, origin))
    build_s = time.perf_counter() - t0
    predictor = Predictor()
    for op in ops:
        state = torch.random.get_rng_state()
        torch.manual_seed(workloads.WEIGHT_SEED[op])
        pred = RuntimePredictor(op, 8, 1024)
        torch.random.set_rng_state(state)
        pred.mu, pred.sigma = workloads.sweep_mu_sigma(op)
        setattr(predictor, op + "_pred", pred)
    trace = Trace(origin, operations)
    dests = ctx.bench_devs[1:]
    with torch.cuda.stream(ctx.stream):
        t0 = time.perf_counter()
        first = trace.to_devices(dests, predictor)
        totals = [t.run_time_ms for t in first]
        first_s = time.perf_counter() - t0
        t0 = time.perf_counter()
        again = trace.to_devices(dests, predictor)
        totals2 = [t.run_time_ms for t in again]
        again_s = time.perf_counter() - t0
        t0 = time.perf_counter()
        touched = sum(op.run_time_ms for op in again[0].operations)        # materialises every operation
        touch_s = time.perf_counter() - t0
    n = len(operations)
    return {"operations": n, "destinations": len(dests), "build_trace_objects_s": build_s,
            "first_prediction_s": first_s, "repeat_prediction_s": again_s,
            "us_per_operation_and_destination": 1e6 * again_s / (n * len(dests)),
            "materialise_one_destination_s": touch_s,
            "totals_agree": bool(totals == totals2 and abs(touched - totals2[0]) <= 1e-9 * totals2[0])}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the cpu_baseline leg and the oracle checks")
    ap.add_argument("--cpu-seconds", type=float, default=0.0,
                    help="reference arm: seconds of CPU work per step and phase (default: sized to the step count)")
    ap.add_argument("--totals", default="peer", choices=["peer", "nccl"],
                    help="how the per-step totals are summed across GPUs")
    ap.add_argument("--case", default="all",
                    choices=["all", "config2", "config2-large", "config2-totals", "sweep-kernel", "config2-status", "config2-regs", "config2-metrics",
                             "config3", "config1"],
                    help="run one kernel-only sub-entry alone and print it (for profilers)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    ctx = Ctx(args)
    torch = ctx.torch
    if args.case != "all":
        if ctx.rank == 0:
            fn = {"config2": lambda: case_config2(ctx, large=False),
                  "config2-large": lambda: case_config2(ctx, small=False),
                  "config2-totals": lambda: case_config2_totals(ctx),
                  "sweep-kernel": lambda: case_sweep_kernel(ctx),
                  "config2-status": lambda: case_config2_inputs(ctx, "status"),
                  "config2-regs": lambda: case_config2_inputs(ctx, "regs"),
                  "config2-metrics": lambda: case_config2_inputs(ctx, "metrics"),
                  "config3": lambda: case_config3(ctx), "config1": lambda: case_config1(ctx)}[args.case]
            print(json.dumps(fn()), flush=True)
        return

    from habitat_b200 import workloads
    rank, world, peaks = ctx.rank, ctx.world, ctx.peaks
    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()
    steps, warm = args.steps, args.warmup
    pairs_total = workloads.SWEEP_KERNELS * WAVE_D
    queries_total = workloads.SWEEP_QUERIES * len(workloads.SWEEP_OPS)

    with torch.cuda.stream(ctx.stream):
        sw = Sweep(ctx, steps + warm)
        ctx.barrier()                 # ranks meet on the host before the first exchange between GPUs
        exchange_check = None
        for i in range(warm):
            # the first warm-up step always takes NCCL: its totals check the peer exchange of the others
            sw.step(i, timed=False, via="nccl" if (i == 0 and world > 1) else None)
        for h in sw.handles.values():
            h.check_status()          # a launch that gave up on a device-side wait ends the run here
        if ctx.totals_via == "peer":
            bad = 0.0
            try:
                ctx.peer.check_status()
                t = sw.totals[:warm].cpu().numpy()
                rel = np.abs(t[1:] - t[0]) / np.abs(t[0])
                exchange_check = float(rel.max())
                if not (rel.max() <= 1e-12):
                    bad = 1.0
            except Exception as exc:                       # noqa: BLE001 - a wait that ran out, or NaN totals
                print("peer exchange failed its warm-up check on rank %d: %s" % (rank, exc), file=sys.stderr)
                bad = 1.0
            flag = torch.tensor([bad], device="cuda")
            ctx.dist.all_reduce(flag, op=ctx.dist.ReduceOp.MAX)
            if float(flag.item()) != 0.0:
                ctx.totals_via = "nccl"                    # every rank falls back together
        def timed_region():
            sw.ev.clear()
            ctx.barrier()
            sampler.mark("timed_start")
            t0, t1 = ctx.event(), ctx.event()
            before = ctx.launches
            t0.record(ctx.stream)
            for i in range(steps):
                sw.step(warm + i)
            t1.record(ctx.stream)
            ctx.barrier()
            sampler.mark("timed_end")
            return ctx.launches - before, t0.elapsed_time(t1)

        timed_launches, total_ms = timed_region()
        tot_host = sw.totals.cpu().numpy()
        fallback_reason = None
        if ctx.totals_via == "peer":
            # a wait for a peer that ran out (NaN totals, status word set) on any rank: every rank
            # repeats the timed region with NCCL all-reduces
            bad = 0.0
            try:
                ctx.peer.check_status()
                if not np.isfinite(tot_host[warm:]).all():
                    bad = 1.0
            except Exception as exc:                       # noqa: BLE001
                print("peer exchange failed in the timed steps on rank %d: %s" % (rank, exc), file=sys.stderr)
                bad = 1.0
            flag = torch.tensor([bad], device="cuda")
            ctx.dist.all_reduce(flag, op=ctx.dist.ReduceOp.MAX)
            if float(flag.item()) != 0.0:
                fallback_reason = "a wait of the peer exchange ran out during the timed steps; they were repeated with NCCL"
                ctx.totals_via = "nccl"
                timed_launches, total_ms = timed_region()
                tot_host = sw.totals.cpu().numpy()
        total_ms = ctx.reduce(total_ms)
        w_ms, k_ms, m_ms, per_op_ms = sw.phase_ms()
        w_ms, m_ms = ctx.reduce(w_ms), ctx.reduce(m_ms)
        for h in sw.handles.values():
            h.check_status()
        same_every_step = bool((tot_host[warm:] == tot_host[warm]).all())

        shard_pairs = (sw.khi - sw.klo) * WAVE_D
        kern_us = 1e3 * k_ms / steps
        achieved = shard_pairs * WAVE_BYTES_PER_PAIR / (kern_us * 1e-6) / 1e9
        nq = sw.qhi - sw.qlo
        mlp_kernel_ms = sum(per_op_ms) / steps
        mlp_flops = sum(nq * mlp_flops_per_query(len(workloads.OP_FEATURES[op])) for op in sw.ops)
        tflops = mlp_flops / (mlp_kernel_ms * 1e-3) / 1e12

        e2e = e2e_sweep(ctx, sw)

    line = {
        "metric": "wave_scaled_kernel_pairs_per_sec", "value": pairs_total * steps / (w_ms * 1e-3),
        "unit": "pairs/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": total_ms / steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "i32+f32", "data": "synthetic",
        "config": {
            "workload": SWEEP_WORKLOAD,
            "step": "one pass over the whole batch: a wave-scaling phase (the table kernel on the rank's kernels, "
                    "whose blocks add up their own results; a final stage over the block sums that ends in the "
                    "all-reduce of the [6] totals) and an MLP phase (the four predictors "
                    "on the rank's queries, per-device totals of each, all-reduce of the [4 x 6] totals); `value` "
                    "is pairs over the wave-scaling phases, `mlp.value` predictions over the MLP phases, "
                    "`ms_per_step` the whole step, all max over ranks, CUDA events on the launching stream",
            "kernels_per_gpu": sw.khi - sw.klo, "queries_per_gpu_and_predictor": nq, "destinations": WAVE_D,
            "l2": "a 256 MB buffer is overwritten before every step, so no step finds its records or its "
                  "outputs of the step before in the 126 MB L2",
            "collective": {"none": "none",
                           "nccl": "two NCCL all-reduces per step (float64 [6] and [24])",
                           "peer": "the final stage of every reduction stores its totals into mailboxes in the peer "
                                   "GPUs' memory and adds up what the peers stored (five exchanges per step: [6] pair "
                                   "totals, 4 x [6] query totals), checked against NCCL all-reduces in the warm-up"
                           }[ctx.totals_via],
            "peer_vs_nccl_max_rel_diff": exchange_check, "collective_fallback": fallback_reason,
            "wave_phase_ms_per_step": w_ms / steps, "mlp_phase_ms_per_step": m_ms / steps,
            "e2e": "the rank's shard from pinned host memory through the host pipelines: one 20 B/kernel block up "
                   "and the predicted times (4 B/pair) down per 1,048,576-kernel chunk; features up (4 F + 1 B per "
                   "query) and predictions down (4 B) per 262,144-query chunk; three chunks in flight"},
        "roofline": {"bound": "hbm", "kernel": "wave_scale_lut_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                     "us_per_launch": kern_us, "kernels_per_launch": sw.khi - sw.klo,
                     "algorithmic_bytes_per_pair": WAVE_BYTES_PER_PAIR,
                     "timing": "CUDA events around the kernel inside the timed steps (rank 0)",
                     "instance": "the one whose blocks also add up their own results per destination (11 % more "
                                 "instructions than the plain instance timed under config2; in exchange no second "
                                 "pass over the predicted times)",
                     "traffic": None},
        "e2e": {"value": pairs_total / (e2e["wave_ms"] * 1e-3), "unit": "pairs/s",
                "h2d_bytes_per_step": workloads.SWEEP_KERNELS * 20, "d2h_bytes_per_step": pairs_total * 4,
                "copy_rates": e2e["copy"],
                "totals_only": {"value": pairs_total / (e2e["totals_ms"] * 1e-3), "unit": "pairs/s",
                                "what": "the same pass for a caller that wants only the per-destination totals of "
                                        "each chunk back (the kernel's blocks add up their own results; nothing "
                                        "else is downloaded)",
                                "h2d_bytes_per_step": workloads.SWEEP_KERNELS * 20,
                                "d2h_bytes_per_step_per_rank": e2e["totals_d2h"],
                                "chunk_totals_vs_device_totals_max_rel_diff": e2e["totals_rel"]}},
        "totals_identical_every_step": same_every_step,
    }
    mlp = {
        "metric": "mlp_predictions_per_sec", "value": queries_total * steps / (m_ms * 1e-3), "unit": "predictions/s",
        "ms_per_step": m_ms / steps, "dtype": "bf16",
        "config": {"workload": "the MLP phase of the same steps: conv2d, linear, bmm and lstm predictors (8 x 1024 "
                               "hidden), 4,194,304 queries each, bf16 tensor cores, fp32 accumulate",
                   "l2": "weights (16.5 MB of bf16 tiles per predictor) stay in L2 by design; the kernel is "
                         "tensor-bound"},
        "roofline": {"bound": "tensor", "kernel": "mlp_chain_pair_kernel", "achieved": tflops,
                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tflops / peaks["bf16_tflops"],
                     "frac_of_sustained": tflops / peaks["bf16_tflops_sustained"], "peak_source": peaks["source"],
                     "ms_per_launch": {op: per_op_ms[j] / steps for j, op in enumerate(sw.ops)},
                     "timing": "CUDA events around each of the four launches inside the timed steps (rank 0)",
                     "traffic": None},
        "e2e": {"value": queries_total / (e2e["mlp_ms"] * 1e-3), "unit": "predictions/s",
                "h2d_bytes_per_step": sum(workloads.SWEEP_QUERIES * (4 * len(workloads.OP_FEATURES[op]) + 1)
                                          for op in workloads.SWEEP_OPS),
                "d2h_bytes_per_step": queries_total * 4},
    }

    # ---- sub-entries: the single-GPU configurations, kernel-only (rank 0; the others wait on the host) ----
    if rank == 0:
        line["roofline"]["config2"] = case_config2(ctx)
        line["roofline"]["config2"]["analyzer_inputs"] = [case_config2_inputs(ctx, m) for m in ("status", "regs", "metrics")]
        mlp["roofline"]["config3"] = case_config3(ctx)
        mlp["split_precision"] = case_config1(ctx)
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel from the ncu
        # captures summarised under profiles/ (per kernel and workload), scaled to this launch by its units
        tr = traffic_from_profiles()
        if tr.get("wave_bytes_per_kernel") is not None:
            line["roofline"]["traffic"] = tr["wave_bytes_per_kernel"] * (sw.khi - sw.klo)
            line["roofline"]["traffic_source"] = tr["wave_source"]
        if tr.get("split_bytes_per_query") is not None:
            mlp["split_precision"]["roofline"]["traffic"] = tr["split_bytes_per_query"] * CONFIG1_Q
            mlp["split_precision"]["roofline"]["traffic_source"] = tr["split_source"]
        if tr.get("mlp_bytes_per_query") is not None:
            mlp["roofline"]["traffic"] = tr["mlp_bytes_per_query"] * nq
            mlp["roofline"]["traffic_source"] = tr["mlp_source"]
    ctx.hd.host_barrier()

    # ---- multi-GPU result check: the all-reduced totals against one GPU working alone ----
    check = {"ranks": world}
    if rank == 0:
        reduced = tot_host[-1]
        if world > 1:
            alone = sweep_totals_alone(ctx, 0, workloads.SWEEP_KERNELS, 0, workloads.SWEEP_QUERIES, sw.handles)
            check["compared"] = "all-reduced totals of %d ranks against the whole batch on rank 0 alone" % world
        else:
            # one GPU: the same batch as two shards summed on the host (the shard bookkeeping of two ranks)
            k1 = ctx.hd.shard_bounds_aligned(workloads.SWEEP_KERNELS, 0, 2, 2)
            q1 = ctx.hd.shard_bounds_aligned(workloads.SWEEP_QUERIES, 0, 2, 128)
            alone = sweep_totals_alone(ctx, k1[0], k1[1], q1[0], q1[1], sw.handles) + \
                sweep_totals_alone(ctx, k1[1], workloads.SWEEP_KERNELS, q1[1], workloads.SWEEP_QUERIES, sw.handles)
            check["compared"] = "totals of the whole batch against the sum of two half-batch shards on the same GPU"
        rel = np.abs(reduced - alone) / np.abs(alone)
        check["max_rel_diff"] = float(rel.max())
        check["totals_match_rtol_1e-12"] = bool(rel.max() <= 1e-12)
        check["wave_totals_ns"] = [float(x) for x in reduced[:WAVE_D]]
    ctx.hd.host_barrier()

    # ---- config 4: the mixed iteration trace, sharded by iteration, all-gather of the rows ----
    c4 = config4(ctx, {op: sw.handles[op] for op in workloads.ITER_SPECIAL}, cpu_leg=not args.skip_cpu)

    if rank == 0:
        sampler.stop()
        line["clocks"] = sampler.summary()
        line["gpu_launches"] = timed_launches
        line["gpu_launches_whole_run"] = ctx.launches
        if not args.skip_cpu:
            if world == 1:
                # the timed CPU baseline belongs to the single-GPU run (the box's host cores are the
                # same at every N); the oracle checks below run at every N
                line["cpu_baseline"] = cpu_wave()
                line["cpu_baseline"].pop("seconds"), line["cpu_baseline"].pop("pairs")
                mlp["cpu_baseline"] = cpu_mlp()
                mlp["cpu_baseline"].pop("seconds"), mlp["cpu_baseline"].pop("queries")
            check["oracle_subset"] = oracle_subset_check(ctx, sw)
        line["mlp"] = mlp
        line["multi_gpu_check"] = check
        line["config4"] = c4
        print(json.dumps(line), flush=True)
    # the other ranks wait for rank 0's host work on a socket, not in a NCCL barrier on their GPUs
    ctx.hd.host_barrier()
    if ctx.peer is not None:
        ctx.peer.close()
    if world > 1:
        ctx.dist.destroy_process_group()


def oracle_subset_check(ctx, sw):
    """cpu_baseline leg: every 64th kernel and query of rank 0's shard against the oracle."""
    from habitat_b200 import workloads
    from oracle import mlp as omlp
    from oracle import wave as owave
    idx = np.arange(0, sw.khi - sw.klo, 64)
    sub = {k: v[idx] for k, v in sw.host_k.items()}
    specs = [d.spec_tuple() for d in ctx.bench_devs]
    ref = owave.wave_scale_batch(specs, 0, list(range(WAVE_D)), sub, want_limits=False)
    t_idx = ctx.torch.from_numpy(idx).cuda()
    got_ns = sw.out.scaled_ns[:, t_idx].cpu().numpy().astype(np.float64)
    got_occ = sw.out.dest_occupancy[:, t_idx].cpu().numpy()
    got_wav = sw.out.dest_waves.view(ctx.torch.int32)[:, t_idx].cpu().numpy().view(np.uint32)
    ok = ref["status"] <= 1
    err = np.abs(got_ns[ok] - ref["scaled_ns"][ok]) / ref["scaled_ns"][ok]
    res = {"kernels_checked": int(len(idx)),
           "integers_exact": bool(np.array_equal(got_occ, ref["dest_occupancy"]) and np.array_equal(got_wav, ref["dest_waves"])
                                  and np.isnan(got_ns[~ok]).all()),
           "scaled_ns_max_rel_err": float(err.max()), "scaled_ns_within_1e-6": bool(err.max() <= 1e-6)}
    worst = 0.0
    nq = 0
    for op in sw.ops:
        feats, dev = sw.host_q[op]
        qi = np.arange(0, len(feats), 64)
        want = omlp.predict(sw.weights[op], feats[qi], dev[qi], workloads.BENCH_DEVICE_FEATURES, *sw.stats[op])
        got = sw.d_o[op][ctx.torch.from_numpy(qi).cuda()].cpu().numpy()
        worst = max(worst, float((np.abs(got - want) / np.abs(want)).max()))
        nq += len(qi)
    res.update({"queries_checked": nq, "mlp_max_rel_err": worst, "mlp_within_2e-2": bool(worst <= 2e-2)})
    return res


def traffic_from_profiles():
    """DRAM bytes of the dominant kernels as measured by ncu, read from the summaries under profiles/
    (a line `dram_bytes_per_kernel: X` / `dram_bytes_per_query: X` in each)."""
    out = {}
    for key, fname, field in (("wave", "wave_scale_lut_kernel__config2.md", "dram_bytes_per_kernel"),
                              ("mlp", "mlp_chain_pair_kernel__config3.md", "dram_bytes_per_query"),
                              ("split", "mlp_chain_pair_kernel__config1_split.md", "dram_bytes_per_query")):
        path = os.path.join(ROOT, "profiles", fname)
        unit = {"wave": "wave_bytes_per_kernel", "mlp": "mlp_bytes_per_query", "split": "split_bytes_per_query"}[key]
        out[unit] = None
        try:
            for ln in open(path):
                if ln.strip().startswith(field + ":"):
                    out[unit] = float(ln.split(":", 1)[1].split()[0])
                    out[key + "_source"] = "profiles/%s (%s, ncu dram__bytes_read.sum + dram__bytes_write.sum " \
                                           "per launch divided by its units)" % (fname, field)
        except OSError:
            pass
    return out


if __name__ == "__main__":
    main()
