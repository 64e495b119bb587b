"""Generates the golden fixtures in this directory from the reference itself.

Run where the reference tree is mounted (HABITAT_REFERENCE_ROOT, default: a `reference`
directory beside this repository):

    python tests/golden/make_golden.py

It imports the reference's own Python modules from where they lie (nothing is
copied) and drives them with seeded inputs:

  wave_scaling.npz  - analyzer/habitat/analysis/wave_scaling/{roofline,resimplified,
                      unified}.py over kernels x (origin, destination) pairs of the
                      reference's devices.yml, through the reference's pybind11
                      bindings compiled into oracle/_ref (KernelInstance factory
                      added by oracle/ref_pybind_shim.cpp); ZeroDivisionError is
                      recorded as NaN; a small kernels.sqlite exercises
                      MetadataManager (wave_scaling/metadata.py);
  mlp_predict.npz   - RuntimePredictor.predict (analysis/mlp/mlp.py:252-267), one
                      call per query, for all four predictors with seeded weights
                      and batch statistics as mu/sigma;
  trace.npz         - Predictor.predict_operation / Trace.to_device
                      (analysis/predictor.py, trace.py) over a small mixed trace.

The reference cannot run on the GPU box (its tree is absent there), which is why
these vectors are committed.  Stand-in data files (checkpoints, kernels.sqlite)
are written to a temporary directory; the reference's import-time
`Trace.DefaultPredictor = Predictor()` reads them from there.
"""
import importlib.util
import os
import sqlite3
import sys
import tempfile
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("HABITAT_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
os.environ["TORCH_FORCE_NO_WEIGHTS_ONLY_LOAD"] = "1"   # the checkpoints hold numpy arrays

import torch  # noqa: E402

from oracle import build as obuild  # noqa: E402


def install_reference(data_dir):
    """Makes `import habitat.analysis...` resolve to the reference tree without
    running its top-level __init__ (which pulls in the CUPTI-based tracker)."""
    outs = obuild.build_ref()
    pkg = types.ModuleType("habitat")
    pkg.__path__ = [os.path.join(REF, "analyzer", "habitat")]
    sys.modules["habitat"] = pkg
    spec = importlib.util.spec_from_file_location("habitat.habitat_cuda", outs["pybind"])
    hc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(hc)
    sys.modules["habitat.habitat_cuda"] = hc
    pkg.habitat_cuda = hc
    data = types.ModuleType("habitat.data")
    ref_data = os.path.join(REF, "analyzer", "habitat", "data")

    def path_to_data(name):
        return os.path.join(ref_data if name == "devices.yml" else data_dir, name)

    data.path_to_data = path_to_data
    sys.modules["habitat.data"] = data
    pkg.data = data
    return hc


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


KERNEL_NAMES = ["volta_sgemm_128x64_nn", "elementwise_kernel", "cudnn_winograd", "reduce_kernel"]


def make_wave_scaling(hc, data_dir):
    from habitat.analysis import Device
    from habitat.analysis.kernels import MeasuredKernel
    from habitat.analysis.metrics import Metric
    from habitat.analysis.wave_scaling.metadata import MetadataManager
    from habitat.analysis.wave_scaling.resimplified import resimplified_wave_scaling
    from habitat.analysis.wave_scaling.roofline import roofline_wave_scaling
    from habitat.analysis.wave_scaling.unified import unified_wave_scaling

    names = ["P4000", "GTX1080Ti", "RTX2070", "RTX2080Ti", "P4", "T4", "V100", "P100"]
    devices = [getattr(Device, n) for n in names]
    meta = MetadataManager(os.path.join(data_dir, "kernels.sqlite"))
    g = rng(20240)
    K = 192
    nb = np.clip(np.floor(np.exp(g.uniform(0, np.log(2 ** 20 + 1), K))), 1, 2 ** 20).astype(np.int32)
    bs = g.choice([32, 64, 96, 128, 256, 512, 1024], K).astype(np.int32)
    regs = g.integers(8, 129, K).astype(np.int32)
    regs[:6] = [0, 255, 256, 64, 65, 128]
    dyn = (256 * g.integers(0, 120, K)).astype(np.int32)
    dyn[g.integers(0, 2, K) == 0] = 0
    static = (g.integers(0, 3, K) == 0) * g.integers(0, 20000, K)
    static = static.astype(np.int32)
    t_ns = np.clip(np.floor(np.exp(g.uniform(np.log(2e3), np.log(5e7), K))), 2000, 5e7).astype(np.int64)
    eff = g.uniform(0, 80, K)
    rd = np.floor(np.exp(g.uniform(np.log(1e3), np.log(1e10), K)))
    wr = np.floor(np.exp(g.uniform(np.log(1e3), np.log(1e10), K)))
    kind = g.integers(0, 16, K)
    eff[kind == 0] = 0.0
    rd[kind == 1] = 0.0
    wr[kind == 1] = 0.0
    has = (g.integers(0, 4, K) != 0)
    name_idx = g.integers(0, len(KERNEL_NAMES), K)

    D = len(devices)
    out = {s: np.full((D, D, K), np.nan) for s in ("roofline", "resimplified", "unified")}
    occupancy = np.zeros((D, K), np.int32)
    for o, (oname, origin) in enumerate(zip(names, devices)):
        legacy = origin.compute_capability[0] < 7
        for k in range(K):
            metrics = []
            if has[k]:
                m = [Metric.SinglePrecisionFLOPEfficiency, Metric.DRAMReadBytes, Metric.DRAMWriteBytes]
                metrics = [((mm.value.legacy_cupti_name if legacy else mm.value.cupti_name), float(v))
                           for mm, v in zip(m, (eff[k], rd[k], wr[k]))]
            c = hc.make_kernel(KERNEL_NAMES[name_idx[k]], int(nb[k]), int(bs[k]), int(dyn[k]),
                               int(static[k]), int(regs[k]), int(t_ns[k]), metrics)
            mk = MeasuredKernel(c, [c] if metrics else [], origin)
            occupancy[o, k] = c.thread_block_occupancy(origin)
            for d, dest in enumerate(devices):
                for sname, fn in (("roofline", roofline_wave_scaling),
                                  ("resimplified", resimplified_wave_scaling),
                                  ("unified", unified_wave_scaling)):
                    try:
                        out[sname][o, d, k] = fn(mk, origin, dest, meta).run_time_ns
                    except ZeroDivisionError:
                        pass
                    except AttributeError:
                        assert sname == "roofline" and not has[k]
    np.savez_compressed(
        os.path.join(HERE, "wave_scaling.npz"), device_names=np.array(names), num_blocks=nb,
        block_size=bs, regs=regs, dynamic_smem=dyn, static_smem=static, run_time_ns=t_ns,
        flop_efficiency=eff, dram_read=rd, dram_write=wr, has_metrics=has.astype(np.uint8),
        kernel_name_index=name_idx.astype(np.int32), kernel_names=np.array(KERNEL_NAMES),
        occupancy=occupancy, roofline=out["roofline"], resimplified=out["resimplified"],
        unified=out["unified"], metadata_rows=np.array(METADATA_ROWS, dtype=object))


METADATA_ROWS = [("volta_sgemm_128x64_nn", 61, 96), ("volta_sgemm_128x64_nn", 70, 120),
                 ("elementwise_kernel", 60, 16), ("elementwise_kernel", 75, 24),
                 ("cudnn_winograd", 70, 255)]


def write_data_files(data_dir):
    from habitat.analysis.mlp.mlp import RuntimePredictor
    con = sqlite3.connect(os.path.join(data_dir, "kernels.sqlite"))
    con.execute("CREATE TABLE kernels (name TEXT, arch INT, registers_per_thread INT, "
                "PRIMARY KEY (name, arch))")
    con.executemany("INSERT INTO kernels VALUES (?, ?, ?)", METADATA_ROWS)
    con.commit()
    con.close()
    from habitat_b200 import workloads
    stats = {}
    for op, seed in workloads.WEIGHT_SEED.items():
        torch.manual_seed(seed)
        pred = RuntimePredictor(op, 8, 1024)
        feats, dev = workloads.make_queries(op, 4096, 500 + seed)
        # device features of the reference's own devices.csv rows
        from habitat.analysis.mlp.devices import get_all_devices
        table = get_all_devices(pred.device_params)
        dn = sorted(table)
        rows = np.array([table[n] for n in dn], dtype=np.float64)
        x = np.concatenate([feats.astype(np.float64), rows[dev % len(dn)]], axis=1)
        pred.mu, pred.sigma = x.mean(axis=0), x.std(axis=0)
        os.makedirs(os.path.join(data_dir, op), exist_ok=True)
        pred.save_state(os.path.join(data_dir, op, "model.pth"))
        stats[op] = (pred.mu, pred.sigma, dn)
    return stats


def make_mlp(data_dir, stats):
    from habitat.analysis.mlp.mlp import RuntimePredictor
    from habitat_b200 import workloads
    save = {}
    for op, seed in workloads.WEIGHT_SEED.items():
        pred = RuntimePredictor(op, 8, 1024, os.path.join(data_dir, op, "model.pth"))
        mu, sigma, dn = stats[op]
        feats, dev = workloads.make_queries(op, 96, 900 + seed)
        dev = dev % len(dn)
        out = np.array([pred.predict([float(v) for v in feats[i]], dn[dev[i]]) for i in range(len(feats))])
        save[op + "_features"] = feats
        save[op + "_device"] = np.array([dn[d] for d in dev])
        save[op + "_prediction"] = out
        save[op + "_mu"] = mu
        save[op + "_sigma"] = sigma
        save[op + "_weight_seed"] = np.int64(seed)
    np.savez_compressed(os.path.join(HERE, "mlp_predict.npz"), **save)


def make_trace(hc, data_dir):
    from habitat.analysis import Device
    from habitat.analysis.arguments import Arguments
    from habitat.analysis.kernels import MeasuredKernel
    from habitat.analysis.metrics import Metric
    from habitat.analysis.operation import MeasuredOperation
    from habitat.analysis.predictor import Predictor
    from habitat.analysis.run_time import RunTimeMeasurement
    from habitat.analysis.trace import Trace

    origin = Device.V100
    g = rng(777)
    ops, spec = [], []

    def kernels(n, with_metrics):
        ks, rec = [], []
        for _ in range(n):
            nb = int(np.floor(np.exp(g.uniform(0, np.log(2 ** 16)))))
            bs = int(g.choice([64, 128, 256, 512]))
            regs = int(g.integers(16, 64))
            dyn = int(256 * g.integers(0, 32))
            t = int(np.floor(np.exp(g.uniform(np.log(2e3), np.log(5e6)))))
            # cudnn_winograd has a 255-register metadata row that cannot launch with
            # these block sizes on cc >= 7.0: the reference raises on it (covered by
            # wave_scaling.npz), so the trace leaves it out
            name = [KERNEL_NAMES[0], KERNEL_NAMES[1], KERNEL_NAMES[3]][int(g.integers(0, 3))]
            metrics = []
            if with_metrics:
                vals = (float(g.uniform(0, 60)), float(np.floor(np.exp(g.uniform(8, 20)))),
                        float(np.floor(np.exp(g.uniform(8, 20)))))
                metrics = [(m.value.cupti_name, v) for m, v in zip(
                    (Metric.SinglePrecisionFLOPEfficiency, Metric.DRAMReadBytes, Metric.DRAMWriteBytes), vals)]
            c = hc.make_kernel(name, nb, bs, dyn, 0, regs, t, metrics)
            ks.append(MeasuredKernel(c, [c] if metrics else [], origin))
            rec.append((name, nb, bs, dyn, 0, regs, t, [m[1] for m in metrics]))
        return ks, rec

    def run(n, with_metrics):
        ks, rec = kernels(n, with_metrics)
        ms = sum(k.run_time_ns for k in ks) / 1e6 + float(g.uniform(-0.001, 0.02))
        return RunTimeMeasurement(ms, ks, origin), (ms, rec)

    for i in range(24):
        kind = i % 6
        if kind in (0, 1, 2):
            f, fr = run(int(g.integers(1, 5)), with_metrics=kind != 2)
            b, br = (run(int(g.integers(1, 4)), with_metrics=kind == 0) if kind != 1 else (None, None))
            ops.append(MeasuredOperation("relu" if kind else "add", Arguments((), {}), f, b, origin))
            spec.append(("wave", fr, br))
        elif kind == 3:
            args = Arguments(((int(g.integers(1, 64)), int(g.integers(3, 512)), int(g.integers(7, 224)), 0),
                              (int(g.integers(3, 512)), 0, int(g.choice([1, 3, 5])), 0), None,
                              (int(g.choice([1, 2])),) * 2, (int(g.integers(0, 3)),) * 2, (1, 1), 1), {})
            ms = float(g.uniform(0.05, 20))
            ops.append(MeasuredOperation("conv2d", args, RunTimeMeasurement(ms, [], origin), None, origin))
            spec.append(("conv2d", args.args, ms))
        elif kind == 4:
            args = Arguments(((int(g.integers(1, 32)), int(g.integers(1, 50)), int(g.integers(16, 4096))),
                              (int(g.integers(16, 4096)), 0), (1,)), {})
            args = Arguments((args.args[0], (args.args[1][0], args.args[0][2]), args.args[2]), {})
            ms = float(g.uniform(0.05, 20))
            ops.append(MeasuredOperation("linear", args, RunTimeMeasurement(ms, [], origin), None, origin))
            spec.append(("linear", args.args, ms))
        else:
            b_, l_, m_, r_ = (int(g.integers(1, 128)), int(g.integers(1, 1024)), int(g.integers(1, 1024)),
                              int(g.integers(1, 1024)))
            args = Arguments(((b_, l_, m_), (b_, m_, r_)), {})
            ms = float(g.uniform(0.05, 20))
            ops.append(MeasuredOperation("bmm", args, RunTimeMeasurement(ms, [], origin), None, origin))
            spec.append(("bmm", args.args, ms))
    # one LSTM of each overload (predictor.py:240-277)
    lstm_a = Arguments(((35, 20, 650), ((2, 20, 650), (2, 20, 650)), [], True, 2, 0.5, True, False, False), {})
    ops.append(MeasuredOperation("lstm", lstm_a, RunTimeMeasurement(3.25, [], origin), None, origin))
    spec.append(("lstm", lstm_a.args, 3.25, None))
    lstm_b = Arguments(((700, 512), (20, 20, 18, 15), ((1, 20, 256), (1, 20, 256)), [], True, 1, 0.0, True, True), {})
    lstm_b.special["batch_sizes"] = [20, 20, 18, 15]
    ops.append(MeasuredOperation("lstm", lstm_b, RunTimeMeasurement(1.5, [], origin), None, origin))
    spec.append(("lstm", lstm_b.args, 1.5, [20, 20, 18, 15]))

    trace = Trace(origin, ops)
    predictor = Predictor(os.path.join(data_dir, "kernels.sqlite"))
    dests = ["T4", "P100", "RTX2080Ti", "P4000", "V100"]
    per_op = np.zeros((len(dests), len(ops)))
    totals = np.zeros(len(dests))
    for d, name in enumerate(dests):
        pt = trace.to_device(getattr(Device, name), predictor)
        per_op[d] = [op.run_time_ms for op in pt.operations]
        totals[d] = pt.run_time_ms
    np.savez_compressed(os.path.join(HERE, "trace.npz"), spec=np.array(spec, dtype=object),
                        dests=np.array(dests), per_op_ms=per_op, total_ms=totals)


def main():
    with tempfile.TemporaryDirectory() as data_dir:
        hc = install_reference(data_dir)
        stats = write_data_files(data_dir)
        make_wave_scaling(hc, data_dir)
        make_mlp(data_dir, stats)
        make_trace(hc, data_dir)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
