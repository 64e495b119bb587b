"""Times the reference's own Python prediction path on this machine's CPU.

Run where the reference tree is mounted (HABITAT_REFERENCE_ROOT, default: a `reference`
directory beside this repository):

    python tests/golden/time_reference.py

It imports the reference's modules from where they lie (as make_golden.py does) and times
  * RuntimePredictor.predict (analysis/mlp/mlp.py:252-267), one call per query, over the
    first 2,048 linear-predictor queries of the benchmark's batch;
  * Trace.to_device (analysis/trace.py:38-51 over predictor.py:111-130) over a trace of
    13,108 single-kernel operations (origin V100) to each of the five other rows the
    reference's devices.yml shares with the benchmark's device classes = 65,540 pairs.
Kernels are rejection-sampled so that the origin can run them (the reference raises
ZeroDivisionError otherwise).  The reference cannot travel to a GPU box, so this is not part
of any test or benchmark; its figures are quoted in the project's notes.
"""
import json
import os
import sys
import tempfile
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import make_golden as mg  # noqa: E402  (sets up sys.path and the reference import hooks)


def main():
    with tempfile.TemporaryDirectory() as data_dir:
        hc = mg.install_reference(data_dir)
        mg.write_data_files(data_dir)
        from habitat.analysis import Device
        from habitat.analysis.arguments import Arguments
        from habitat.analysis.kernels import MeasuredKernel
        from habitat.analysis.mlp.mlp import RuntimePredictor
        from habitat.analysis.operation import MeasuredOperation
        from habitat.analysis.predictor import Predictor
        from habitat.analysis.run_time import RunTimeMeasurement
        from habitat.analysis.trace import Trace
        from habitat_b200 import workloads
        import torch

        out = {"cores": os.cpu_count(), "torch_threads": torch.get_num_threads()}
        pred = RuntimePredictor("linear", 8, 1024, os.path.join(data_dir, "linear", "model.pth"))
        feats, _ = workloads.sweep_queries("linear", 0, 2048)
        names = ["V100", "T4", "P100", "P4000", "RTX2070", "RTX2080Ti"]
        pred.predict([float(v) for v in feats[0]], "V100")
        t = time.perf_counter()
        for i in range(len(feats)):
            pred.predict([float(v) for v in feats[i]], names[i % len(names)])
        dt = time.perf_counter() - t
        out["predict_calls"] = len(feats)
        out["predict_s"] = dt
        out["predictions_per_s"] = len(feats) / dt

        origin = Device.V100
        n = 13108

        def occ(block, smem, regs):
            return np.array([hc.make_kernel("k", 1, int(b), int(s), 0, int(r), 1000, []).thread_block_occupancy(origin)
                             for b, s, r in zip(block, smem, regs)])
        k = workloads.make_kernels(n, 1002, valid_only=True, origin=occ)
        ops = []
        for i in range(n):
            c = hc.make_kernel("kernel_%d" % (i % 16), int(k["num_blocks"][i]), int(k["block_size"][i]),
                               int(k["smem_bytes"][i]), 0, int(k["regs_per_thread"][i]), int(k["run_time_ns"][i]), [])
            run = RunTimeMeasurement(float(k["run_time_ns"][i]) / 1e6 + 0.005, [MeasuredKernel(c, [], origin)], origin)
            ops.append(MeasuredOperation("relu", Arguments((), {}), run, None, origin))
        trace = Trace(origin, ops)
        predictor = Predictor()
        dests = [getattr(Device, d) for d in names[1:]]
        t = time.perf_counter()
        totals = [trace.to_device(d, predictor).run_time_ms for d in dests]
        dt = time.perf_counter() - t
        out["wave_pairs"] = n * len(dests)
        out["to_device_s"] = dt
        out["pairs_per_s"] = n * len(dests) / dt
        out["us_per_pair"] = 1e6 * dt / (n * len(dests))
        out["totals_ms"] = totals
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
