#!/usr/bin/env python
"""Benchmark of the batched prediction path: wave-scaled kernel pairs/s and MLP predictions/s.

One JSON line on stdout (rank 0).  The headline `value` is wave-scaled
(kernel x destination) pairs per second on the 1,048,576-kernel x 6-device
workload; the `mlp` object carries predictions per second of the fused conv2d
predictor on 262,144 queries.  Both are measured three ways: on the device with
inputs resident in HBM (`value`), end to end from pinned host buffers through
the public API (`e2e`), and on the host cores with the CPU oracle
(`cpu_baseline`).  `--impl reference` times only the CPU implementation.

Multi-GPU (torchrun, one rank per GPU): every rank processes its own batch of
the same size (weak scaling); the only exchange is one NCCL all-reduce of the
per-step per-destination totals at the end of the timed region.
"""
import argparse
import json
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

WAVE_K = 1 << 20            # kernels per step and GPU
WAVE_D = 6
WAVE_SETS = 4               # rotating buffer sets: 4 x 79 MB > 126 MB of L2
WAVE_BYTES_PER_PAIR = 25.0 / WAVE_D + 9.0   # 20 B read + 5 B written per kernel, 9 B per pair
MLP_Q = 262144
MLP_OP = "conv2d"
MLP_FLOPS_PER_QUERY = 2 * ((8 + 4) * 1024 + 8 * 1024 * 1024 + 1024)   # 16,803,840


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


def pinned_inputs(torch, arrays):
    """Kernel records as pinned host tensors (unsigned fields viewed as signed)."""
    out = {}
    for k, v in arrays.items():
        a = np.ascontiguousarray(v.astype(np.float32) if k == "run_time_ns" else v)
        if a.dtype == np.uint16:
            a = a.view(np.int16)
        elif a.dtype == np.uint32:
            a = a.view(np.int32)
        out[k] = torch.from_numpy(a).pin_memory()
    return out


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), \
        int(os.environ.get("WORLD_SIZE", 1))


# ---------------------------------------------------------------------------
# CPU baseline (the oracle; the only place the benchmark executes oracle/)
# ---------------------------------------------------------------------------
def cpu_wave(target_s=8.0, repeats=1):
    """Times the C oracle (OpenMP, all host cores) on a sample sized for about
    `target_s` seconds per pass; `repeats` passes over the same sample."""
    from habitat_b200 import device_table, workloads
    from oracle import wave as owave
    devs = device_table.load_device_file()
    specs = [devs[n].spec_tuple() for n in workloads.BENCH_DEVICES]
    k = workloads.make_kernels(1 << 17, 1002)
    owave.wave_scale_batch(specs, 0, list(range(WAVE_D)), k, want_limits=False)
    t = time.perf_counter()
    r = owave.wave_scale_batch(specs, 0, list(range(WAVE_D)), k, want_limits=False)
    rate = (1 << 17) * WAVE_D / (time.perf_counter() - t)
    n = int(min(max(rate * target_s / WAVE_D, 1 << 17), 1 << 25))
    k = workloads.make_kernels(n, 1002)
    times = []
    for _ in range(repeats):
        t = time.perf_counter()
        r = owave.wave_scale_batch(specs, 0, list(range(WAVE_D)), k, want_limits=False)
        times.append(time.perf_counter() - t)
    dt = float(np.mean(times))
    return {"value": n * WAVE_D / dt, "unit": "pairs/s", "cores": int(r["threads"]), "kind": "port",
            "sample": "%d kernels x %d devices of the same distribution, C oracle under OpenMP, "
                      "%.1f s per pass" % (n, WAVE_D, dt), "seconds": times, "pairs": n * WAVE_D}


def cpu_mlp(target_s=10.0):
    from habitat_b200 import workloads
    from oracle import mlp as omlp
    w = workloads.torch_init_mlp_weights(MLP_OP)
    f, d = workloads.make_queries(MLP_OP, 4096, 1003)
    mu, sg = workloads.batch_mu_sigma(f, d)
    t = time.perf_counter()
    omlp.predict(w, f, d, workloads.BENCH_DEVICE_FEATURES, mu, sg)
    rate = 4096 / (time.perf_counter() - t)
    n = int(min(max(rate * target_s, 4096), MLP_Q))
    f, d = workloads.make_queries(MLP_OP, n, 1003)
    t = time.perf_counter()
    omlp.predict(w, f, d, workloads.BENCH_DEVICE_FEATURES, mu, sg)
    dt = time.perf_counter() - t
    return {"value": n / dt, "unit": "predictions/s", "cores": os.cpu_count(), "kind": "port",
            "sample": "%d conv2d queries, float32 numpy/BLAS forward of the same weights, %.1f s" % (n, dt)}


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    steps = max(1, args.steps)
    per = max(0.5, min(8.0, 90.0 / (steps + args.warmup)))
    wave = cpu_wave(target_s=per, repeats=steps + args.warmup)
    timed = wave.pop("seconds")[args.warmup:]
    wall = float(np.sum(timed))
    wave["value"] = wave.pop("pairs") * len(timed) / wall
    mlp = cpu_mlp(target_s=per)
    line = {
        "impl": "reference", "metric": "wave_scaled_kernel_pairs_per_sec", "value": wave["value"],
        "unit": "pairs/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * wall / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "i32+f64", "data": "synthetic",
        "config": {"workload": "config 2: wave scaling of 1,048,576 synthetic kernels from a "
                               "V100-class origin to 6 device rows, per GPU and step",
                   "sample": "each step a bounded sample of that workload (same distribution, same six "
                             "rows) on the host cores"},
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
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the cpu_baseline leg")
    ap.add_argument("--only", default="both", choices=["both", "wave", "mlp"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist
    from habitat_b200 import batched, device_table, hostio, workloads

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = load_peaks()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    launches = 0
    steps, warm = args.steps, args.warmup
    devs = device_table.load_device_file()
    bench_devs = [devs[n] for n in workloads.BENCH_DEVICES]
    origin = bench_devs[0]
    stream = torch.cuda.Stream()
    line = {}

    with torch.cuda.stream(stream):
        # ------------------------------ wave scaling ------------------------------
        if args.only in ("both", "wave"):
            host_sets = [workloads.make_kernels(WAVE_K, 1002 + 17 * s + 1000 * rank) for s in range(WAVE_SETS)]
            kbs = [batched.KernelBatch.from_numpy(h) for h in host_sets]
            outs = [batched.wave_scale(kbs[s], origin, bench_devs) for s in range(WAVE_SETS)]
            totals = torch.zeros((steps, WAVE_D), dtype=torch.float64, device="cuda")

            def wave_step(i, with_sum=True):
                s = i % WAVE_SETS
                batched.wave_scale(kbs[s], origin, bench_devs, out=outs[s])
                if with_sum:
                    batched.plane_sum(outs[s].scaled_ns, out=totals[i % steps])

            for i in range(warm):
                wave_step(i)
            torch.cuda.synchronize()
            g_full, g_kernel = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            # Timed steps: the totals of step i run on a second stream beside the wave kernel of
            # step i + 1 (a buffer set is reused only after its totals were taken).
            side = torch.cuda.Stream()
            with torch.cuda.graph(g_full, stream=stream):
                waved = [torch.cuda.Event() for _ in range(steps)]
                summed = [torch.cuda.Event() for _ in range(steps)]
                side.wait_stream(stream)
                for i in range(steps):
                    s = i % WAVE_SETS
                    if i >= WAVE_SETS:
                        stream.wait_event(summed[i - WAVE_SETS])
                    batched.wave_scale(kbs[s], origin, bench_devs, out=outs[s])
                    waved[i].record(stream)
                    with torch.cuda.stream(side):
                        side.wait_event(waved[i])
                        batched.plane_sum(outs[s].scaled_ns, out=totals[i % steps])
                        summed[i].record(side)
                stream.wait_stream(side)
            with torch.cuda.graph(g_kernel, stream=stream):
                for i in range(steps):
                    wave_step(i, with_sum=False)
            g_full.replay()
            g_kernel.replay()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            barrier()
            sampler.mark("timed_start")
            ev[0].record(stream)
            g_full.replay()
            if world > 1:
                dist.all_reduce(totals)
            ev[1].record(stream)
            barrier()
            wave_ms = max_over_ranks(ev[0].elapsed_time(ev[1]))
            launches += 3 * steps
            # the dominant kernel alone, same rotation of buffer sets
            ev[2].record(stream)
            g_kernel.replay()
            ev[3].record(stream)
            torch.cuda.synchronize()
            kern_ms = ev[2].elapsed_time(ev[3]) / steps
            wave_kernel = batched.wave_scale_path()     # which kernel the library chose for this launch
            pairs = WAVE_K * WAVE_D
            achieved = pairs * WAVE_BYTES_PER_PAIR / (kern_ms * 1e-3) / 1e9

            # end to end: pinned host buffers in, pinned host buffers out, through the host
            # pipeline of the package (upload + kernel of step i + 1 overlap the download of step i)
            e2e_steps = max(4, min(steps, 12))
            pin_in = [pinned_inputs(torch, h) for h in host_sets[:2]]
            # the step's result on the host: the predicted times [6 x K] (what Predictor._wave_scale
            # returns per kernel); occupancies and wave counts stay on the device
            pipe = hostio.WaveScaleHost(origin, bench_devs, WAVE_K, depth=2, results=("scaled_ns",))
            h2d, d2h = pipe.h2d_bytes, pipe.d2h_bytes
            for i in range(2):
                pipe.submit(pin_in[i % 2], i % 2)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(pipe.s_up)
            for i in range(e2e_steps):
                pipe.submit(pin_in[i % 2], i % 2)
            e1.record(pipe.s_out)
            barrier()
            e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
            del pipe
            line.update({
                "metric": "wave_scaled_kernel_pairs_per_sec",
                "value": world * steps * pairs / (wave_ms * 1e-3), "unit": "pairs/s",
                "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": wave_ms / steps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "i32+f32", "data": "synthetic",
                "config": {"workload": "config 2: wave scaling of 1,048,576 synthetic kernels from a "
                                       "V100-class origin to 6 device rows, per GPU and step",
                           "kernels_per_step_per_gpu": WAVE_K, "destinations": WAVE_D,
                           "l2": "%d rotating buffer sets (%.0f MB) so that no step finds its data in "
                                 "the 126 MB L2" % (WAVE_SETS, WAVE_SETS * pairs * WAVE_BYTES_PER_PAIR / 1e6),
                           "launch": "the timed steps are replayed from one CUDA graph; a step is the "
                                     "wave-scale kernel plus the per-destination totals, the totals of "
                                     "step i on a second stream beside the kernel of step i + 1",
                           "e2e": "pinned host records in (20 B per kernel), predicted times out (4 B per pair), "
                                  "three streams, two batches in flight",
                           "collective": "one all-reduce of the [steps x 6] totals" if world > 1 else "none"},
                "roofline": {"bound": "hbm", "kernel": wave_kernel,
                             "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                             "us_per_launch": kern_ms * 1e3,
                             "algorithmic_bytes_per_pair": WAVE_BYTES_PER_PAIR,
                             # dram__bytes_read + dram__bytes_write of one launch (ncu capture summarised
                             # in profiles/): the 21 MB of input is read; most of the 62 MB of output is
                             # still in the 126 MB L2 when the launch ends
                             "traffic": 28.3e6, "traffic_unit": "bytes per launch (ncu)"},
                "e2e": {"value": world * pairs / (e2e_ms * 1e-3), "unit": "pairs/s",
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            })
            del kbs, outs, pin_in

            # The same kernel on a batch eight times as large (two buffer sets, 1.3 GB): about 4 us of
            # a launch are ramp-up and tail, so the benchmark's 21 us launches understate the rate
            # the kernel sustains.  Reported beside the roofline figure, not instead of it.
            if rank == 0:
                big_k = 8 * WAVE_K
                big = [batched.KernelBatch.from_numpy(workloads.make_kernels(big_k, 7001 + s)) for s in range(2)]
                big_out = [batched.wave_scale(big[s], origin, bench_devs) for s in range(2)]
                torch.cuda.synchronize()
                g_big = torch.cuda.CUDAGraph()
                reps = 6
                with torch.cuda.graph(g_big, stream=stream):
                    for i in range(reps):
                        batched.wave_scale(big[i % 2], origin, bench_devs, out=big_out[i % 2])
                g_big.replay()
                b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                b0.record(stream)
                g_big.replay()
                b1.record(stream)
                torch.cuda.synchronize()
                big_ms = b0.elapsed_time(b1) / reps
                big_gbs = big_k * WAVE_D * WAVE_BYTES_PER_PAIR / (big_ms * 1e-3) / 1e9
                line["roofline"]["large_batch"] = {
                    "kernels": big_k, "us_per_launch": big_ms * 1e3, "achieved": big_gbs,
                    "frac": big_gbs / peaks["hbm_gbs"]}
                del big, big_out, g_big

        # ------------------------------ MLP predictor ------------------------------
        if args.only in ("both", "mlp"):
            w = workloads.torch_init_mlp_weights(MLP_OP)
            feats, dev = workloads.make_queries(MLP_OP, MLP_Q, 1003 + 1000 * rank)
            mu, sigma = workloads.batch_mu_sigma(feats, dev)
            handle = batched.MLPHandle(feats.shape[1], mu=mu, sigma=sigma,
                                       device_features=workloads.BENCH_DEVICE_FEATURES, **w)
            d_f, d_r = torch.from_numpy(feats).cuda(), torch.from_numpy(dev).cuda()
            d_o = torch.empty((MLP_Q,), dtype=torch.float32, device="cuda")
            mtot = torch.zeros((steps, 1), dtype=torch.float64, device="cuda")

            def mlp_step(i):
                handle.predict(d_f, d_r, out=d_o)
                batched.plane_sum(d_o.view(1, -1), out=mtot[i % steps])

            mlp_step(0)
            handle.check_status()      # a launch that gave up on a device-side wait ends the run here
            for i in range(warm):
                mlp_step(i)
            barrier()
            if "metric" not in line:
                sampler.mark("timed_start")
            m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            m0.record(stream)
            for i in range(steps):
                mlp_step(i)
            if world > 1:
                dist.all_reduce(mtot)
            m1.record(stream)
            barrier()
            sampler.mark("timed_end")
            mlp_ms = max_over_ranks(m0.elapsed_time(m1))
            launches += 3 * steps
            handle.check_status()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record(stream)
            for i in range(steps):
                handle.predict(d_f, d_r, out=d_o)
            k1.record(stream)
            torch.cuda.synchronize()
            kern_ms = k0.elapsed_time(k1) / steps
            tflops = MLP_Q * MLP_FLOPS_PER_QUERY / (kern_ms * 1e-3) / 1e12
            # SM clock inside the last launch: cycles and nanoseconds of the MMA issuer's loop
            pc = handle.phase_cycles()
            mlp_sm_mhz = 1e3 * pc["mma_total_cycles"] / pc["mma_total_ns"] if pc["mma_total_ns"] > 0 else None

            p_f, p_r = torch.from_numpy(feats).pin_memory(), torch.from_numpy(dev).pin_memory()
            mpipe = hostio.MLPPredictHost(handle, MLP_Q, depth=2)
            for i in range(2):
                mpipe.submit(p_f, p_r, i % 2)
            barrier()
            e2e_steps = max(4, min(steps, 12))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(mpipe.s_up)
            for i in range(e2e_steps):
                mpipe.submit(p_f, p_r, i % 2)
            e1.record(mpipe.s_out)
            barrier()
            e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
            mlp = {
                "metric": "mlp_predictions_per_sec", "value": world * steps * MLP_Q / (mlp_ms * 1e-3),
                "unit": "predictions/s", "ms_per_step": mlp_ms / steps, "dtype": "bf16",
                "config": {"workload": "config 3: conv2d predictor (8 x 1024 hidden), 262,144 queries per "
                                       "GPU and step, bf16 tensor cores, fp32 accumulate",
                           "l2": "weights (16.5 MB of bf16 tiles) stay in L2 by design; the kernel is "
                                 "tensor-bound, per-query HBM traffic is 37 B"},
                "roofline": {"bound": "tensor", "kernel": "mlp_chain_pair_kernel", "achieved": tflops,
                             "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                             "frac": tflops / peaks["bf16_tflops"],
                             "frac_of_sustained": tflops / peaks["bf16_tflops_sustained"],
                             "peak_source": peaks["source"], "ms_per_launch": kern_ms,
                             "sm_mhz_in_kernel": mlp_sm_mhz,
                             "flops_per_query": MLP_FLOPS_PER_QUERY,
                             # dram__bytes_read + dram__bytes_write of one launch (ncu capture
                             # summarised in profiles/): weights once plus the queries
                             "traffic": 25.8e6, "traffic_unit": "bytes per launch (ncu)"},
                "e2e": {"value": world * MLP_Q / (e2e_ms * 1e-3), "unit": "predictions/s",
                        "h2d_bytes_per_step": int(mpipe.h2d_bytes),
                        "d2h_bytes_per_step": int(mpipe.d2h_bytes)},
            }
            if rank == 0:
                # config 1 beside it: the linear predictor on 65,536 queries in the split-precision mode
                # (the 1e-4 configuration), kernel time only
                w1 = workloads.torch_init_mlp_weights("linear")
                f1, r1 = workloads.make_queries("linear", 65536, 1001)
                mu1, sigma1 = workloads.batch_mu_sigma(f1, r1)
                h1 = batched.MLPHandle(f1.shape[1], mu=mu1, sigma=sigma1, precision="bf16x3",
                                       device_features=workloads.BENCH_DEVICE_FEATURES, **w1)
                d_f1, d_r1 = torch.from_numpy(f1).cuda(), torch.from_numpy(r1).cuda()
                d_o1 = torch.empty((65536,), dtype=torch.float32, device="cuda")
                for _ in range(3):
                    h1.predict(d_f1, d_r1, out=d_o1)
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record(stream)
                for _ in range(5):
                    h1.predict(d_f1, d_r1, out=d_o1)
                c1.record(stream)
                torch.cuda.synchronize()
                h1.check_status()
                ms1 = c0.elapsed_time(c1) / 5
                mlp["split_precision"] = {
                    "workload": "config 1: linear predictor, 65,536 queries, bf16 hi + lo operands (three "
                                "products per step), tolerance 1e-4",
                    "ms_per_launch": ms1, "value": 65536 / (ms1 * 1e-3), "unit": "predictions/s"}
                h1.close()
            if "metric" in line:
                line["mlp"] = mlp
            else:
                line.update(mlp)
                line.update({"n_gpus": world, "steps": steps, "warmup": warm, "higher_is_better": True,
                             "scaling": "weak", "vs_baseline": None, "data": "synthetic"})
        else:
            sampler.mark("timed_end")

    if rank == 0:
        sampler.stop()
        line["clocks"] = sampler.summary()
        line["gpu_launches"] = launches
        if not args.skip_cpu:
            if args.only in ("both", "wave"):
                line["cpu_baseline"] = cpu_wave()
                line["cpu_baseline"].pop("seconds"), line["cpu_baseline"].pop("pairs")
            if args.only in ("both", "mlp"):
                (line["mlp"] if "mlp" in line else line)["cpu_baseline"] = cpu_mlp()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
