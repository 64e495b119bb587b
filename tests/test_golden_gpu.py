"""The CUDA path (through the C ABI and the Python surface) against fixtures produced
by the reference's own Python code (tests/golden/make_golden.py)."""
import os
import sqlite3

import numpy as np
import pytest
import torch

from habitat_b200 import workloads
from habitat_b200.analysis.arguments import Arguments
from habitat_b200.analysis.kernels import MeasuredKernel
from habitat_b200.analysis.metrics import Metric
from habitat_b200.analysis.mlp.mlp import RuntimePredictor
from habitat_b200.analysis.operation import MeasuredOperation
from habitat_b200.analysis.predictor import Predictor
from habitat_b200.analysis.run_time import RunTimeMeasurement
from habitat_b200.analysis.trace import Trace
from habitat_b200.habitat_cuda import KernelInstance
from tests import golden_util as gu
from tests.helpers import run_wave_gpu

pytestmark = pytest.mark.gpu


def _wave_inputs(g):
    kernels = dict(
        num_blocks=g["num_blocks"].astype(np.int32), block_size=g["block_size"].astype(np.uint16),
        regs_per_thread=g["regs"].astype(np.uint16),
        smem_bytes=(g["dynamic_smem"] + g["static_smem"]).astype(np.uint32),
        run_time_ns=g["run_time_ns"].astype(np.float64),
        gamma=np.ones(len(g["num_blocks"]), np.float32))
    metrics = dict(flop_efficiency_pct=g["flop_efficiency"], dram_read_bytes=g["dram_read"],
                   dram_write_bytes=g["dram_write"], has_metrics=g["has_metrics"])
    return kernels, metrics


def _dest_regs(g, devs):
    rows = [tuple(r) for r in g["metadata_rows"]]
    names = [str(n) for n in g["kernel_names"]]
    out = np.empty((len(devs), len(g["num_blocks"])), np.int16)
    for d, dev in enumerate(devs):
        for k, idx in enumerate(g["kernel_name_index"]):
            out[d, k] = gu.metadata_lookup(rows, names[idx], gu.arch_of(dev))
    return out


def _check(got_ns, want, rel):
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got_ns), nan)
    err = np.abs(got_ns[~nan].astype(np.float64) - want[~nan]) / want[~nan]
    assert err.max() <= rel, err.max()


def test_wave_scaling_unified_and_resimplified(device_file):
    g = gu.load("wave_scaling.npz")
    devs = [device_file[str(n)] for n in g["device_names"]]
    kernels, metrics = _wave_inputs(g)
    dest_regs = _dest_regs(g, devs)
    for o, origin in enumerate(devs):
        got = run_wave_gpu(kernels, origin, devs, dest_regs=dest_regs, metrics=metrics)
        _check(got["scaled_ns"], g["unified"][o], 1e-6)
        assert np.array_equal(got["origin_occupancy"], g["occupancy"][o].astype(np.uint8))
        plain = run_wave_gpu(kernels, origin, devs, dest_regs=dest_regs)      # gamma = 1
        _check(plain["scaled_ns"], g["resimplified"][o], 1e-6)
        _check(plain["fast"]["scaled_ns"], g["resimplified"][o], 1e-6)


def _predictor(op, g, precision):
    torch.manual_seed(int(g[op + "_weight_seed"]))
    pred = RuntimePredictor(op, 8, 1024, precision=precision)
    pred.mu, pred.sigma = g[op + "_mu"], g[op + "_sigma"]
    return pred


@pytest.mark.parametrize("op", ["linear", "lstm", "conv2d", "bmm"])
@pytest.mark.parametrize("precision,tol", [("bf16", 2e-2), ("bf16x3", 1e-4)])
def test_mlp_predict_api(op, precision, tol):
    g = gu.load("mlp_predict.npz")
    pred = _predictor(op, g, precision)
    feats, names, want = g[op + "_features"], [str(n) for n in g[op + "_device"]], g[op + "_prediction"]
    for i in range(8):                                    # the scalar API of the reference
        got = pred.predict([float(v) for v in feats[i]], names[i])
        assert isinstance(got, float)
        assert abs(got - want[i]) <= tol * abs(want[i])
    rows = torch.tensor([pred.device_row(n) for n in names], dtype=torch.uint8, device="cuda")
    got = pred.predict_batch(torch.from_numpy(feats).cuda(), rows).cpu().numpy()
    assert (np.abs(got - want) <= tol * np.abs(want)).all()
    with pytest.raises(IndexError):
        pred.predict([float(v) for v in feats[0]], "NoSuchGPU")


def _rebuild_trace(g, origin):
    names = (Metric.SinglePrecisionFLOPEfficiency, Metric.DRAMReadBytes, Metric.DRAMWriteBytes)

    def run(rec):
        if rec is None:
            return None
        ms, ks = rec
        kernels = []
        for name, nb, bs, dyn, static, regs, t, mvals in ks:
            metrics = [(m.value.cupti_name, v) for m, v in zip(names, mvals)]
            c = KernelInstance(name, nb, bs, dyn, static, regs, t, metrics)
            kernels.append(MeasuredKernel(c, [c] if metrics else [], origin))
        return RunTimeMeasurement(ms, kernels, origin)

    ops = []
    for item in g["spec"]:
        kind = item[0]
        if kind == "wave":
            ops.append(MeasuredOperation("relu", Arguments((), {}), run(item[1]), run(item[2]), origin))
        else:
            args = Arguments(tuple(item[1]), {})
            if kind == "lstm" and item[3] is not None:
                args.special["batch_sizes"] = list(item[3])
            ops.append(MeasuredOperation(kind, args, RunTimeMeasurement(item[2], [], origin), None, origin))
    return Trace(origin, ops)


def test_trace_to_device(device_file, tmp_path):
    """Trace.to_device through the analyzer surface: same objects in, predicted
    operations out, per-operation and whole-trace times as the reference gives."""
    g = gu.load("trace.npz")
    w = gu.load("wave_scaling.npz")
    m = gu.load("mlp_predict.npz")
    lut = str(tmp_path / "kernels.sqlite")
    con = sqlite3.connect(lut)
    con.execute("CREATE TABLE kernels (name TEXT, arch INT, registers_per_thread INT)")
    con.executemany("INSERT INTO kernels VALUES (?, ?, ?)", [tuple(r) for r in w["metadata_rows"]])
    con.commit()
    con.close()
    paths = {}
    for op in ("linear", "lstm", "conv2d", "bmm"):
        pred = _predictor(op, m, "bf16")
        os.makedirs(tmp_path / op)
        paths[op] = str(tmp_path / op / "model.pth")
        pred.save_state(paths[op])
    predictor = Predictor(lut, model_paths=paths)
    origin = device_file["V100"]
    trace = _rebuild_trace(g, origin)
    dests = [device_file[str(n)] for n in g["dests"]]
    is_mlp = np.array([item[0] != "wave" for item in g["spec"]])
    for d, dest in enumerate(dests):
        pt = trace.to_device(dest, predictor)
        if dest.name == origin.name:
            assert pt is trace
            continue
        got = np.array([op.run_time_ms for op in pt.operations])
        want = g["per_op_ms"][d]
        assert (np.abs(got - want)[~is_mlp] <= 1e-6 * want[~is_mlp]).all()
        assert (np.abs(got - want)[is_mlp] <= 2e-2 * want[is_mlp]).all()
        assert abs(pt.run_time_ms - g["total_ms"][d]) <= 2e-2 * g["total_ms"][d]
        assert pt.device is dest and len(pt.operations) == len(trace.operations)
        with pytest.raises(RuntimeError):
            pt.operations[0].to_device(origin, predictor)
    # metrics, the register table and the raise-on-NaN rule all ride on the tabulated kernel
    from habitat_b200 import batched
    assert batched.wave_scale_path() == "wave_scale_lut_kernel"
    many = trace.to_devices(dests, predictor)             # all destinations in one pass
    for d, pt in enumerate(many):
        assert abs(pt.run_time_ms - g["total_ms"][d]) <= 2e-2 * g["total_ms"][d]
    # the kernel records were flattened by the first prediction and are reused from the trace
    from habitat_b200.analysis.wave_scaling import batch as wave_batch
    calls = []
    real = wave_batch.flatten_kernels
    wave_batch.flatten_kernels = lambda *a, **k: (calls.append(1), real(*a, **k))[1]
    try:
        again = trace.to_devices(dests, predictor)
    finally:
        wave_batch.flatten_kernels = real
    assert not calls
    for pt, first in zip(again, many):
        assert pt.run_time_ms == first.run_time_ms
