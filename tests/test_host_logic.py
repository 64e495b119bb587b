"""Host-side pieces of the analyzer surface that need no GPU."""
import sqlite3

import numpy as np
import pytest

from habitat_b200 import device_table, workloads
from habitat_b200.analysis import SPECIAL_OPERATIONS, Device
from habitat_b200.analysis.arguments import Arguments
from habitat_b200.analysis.kernels import MeasuredKernel, PredictedKernel
from habitat_b200.analysis.metrics import Metric, resolve_metrics
from habitat_b200.analysis.mlp.devices import get_all_devices, get_device_features
from habitat_b200.analysis.mlp.mlp import RuntimePredictor
from habitat_b200.analysis.operation import MeasuredOperation, PredictedOperation
from habitat_b200.analysis.predictor import (bmm_features, conv2d_features, linear_features,
                                             lstm_features)
from habitat_b200.analysis.run_time import RunTimeMeasurement, RunTimePrediction, RunTimePurePrediction
from habitat_b200.analysis.wave_scaling import batch as wave_batch
from habitat_b200.analysis.wave_scaling.metadata import MetadataManager
from habitat_b200.habitat_cuda import DeviceProperties, KernelInstance
from habitat_b200.utils import ms_to_ns, name_all_arguments, ns_to_ms


def test_device_table_formats(tmp_path):
    devs = device_table.load_device_file()
    assert devs["V100"].num_sms == 80 and devs["V100"].compute_capability == (7, 0)
    assert devs["B200"].spec_tuple()[11] == 1024          # reserved shared memory from cc 8.0 on
    assert Device.T4.mem_bandwidth_gb == 239 and "B200" in Device.names()
    with pytest.raises(KeyError):
        Device.NoSuchGPU
    ref_style = tmp_path / "devices.yml"               # the reference's one-mapping-per-device format
    ref_style.write_text(
        "X1:\n  compute_major: 7\n  compute_minor: 0\n  max_threads_per_block: 1024\n"
        "  max_threads_per_multiprocessor: 2048\n  regs_per_block: 65536\n"
        "  regs_per_multiprocessor: 65536\n  warp_size: 32\n  shared_mem_per_block: 49152\n"
        "  shared_mem_per_multiprocessor: 98304\n  num_sms: 80\n  shared_mem_per_block_optin: 0\n"
        "  mem_bandwidth_gb: 739\n  base_clock_mhz: 1312\n  peak_gflops_per_second: 6716\n")
    x1 = device_table.load_device_file(str(ref_style))["X1"]
    assert x1.spec_tuple() == devs["V100"].spec_tuple()
    with pytest.raises(TypeError):
        DeviceProperties("bad", 7, 0, 1024, 2048, 65536, 65536, 32, 49152, 98304, 80, 0, 739.5, 1312, 6716)


def test_metrics_and_kernels():
    v100, p100 = Device.V100, Device.P100
    assert resolve_metrics([Metric.DRAMReadBytes], v100) == ["dram__bytes_read.sum"]
    assert resolve_metrics(Metric.DRAMReadBytes, p100) == ["dram_read_bytes"]
    assert resolve_metrics(None, v100) == [] and resolve_metrics(["raw"], v100) == ["raw"]
    c = KernelInstance("k", 10, 128, 0, 0, 32, 5000, [("dram_utilization", 3.0), ("dram__bytes_read.sum", 7.0)])
    legacy = MeasuredKernel(c, [c], p100)
    assert legacy.get_metric(Metric.DRAMUtilization) == 30.0      # pre-Volta scale is x10
    assert MeasuredKernel(c, [c], v100).get_metric(Metric.DRAMReadBytes) == 7.0
    with pytest.raises(AttributeError):
        legacy.get_metric(Metric.DRAMWriteBytes)
    assert legacy.get_metric(Metric.DRAMWriteBytes, default=1.5) == 1.5
    assert legacy.num_blocks == 10 and legacy.metadata["registers_per_thread"] == 32   # delegation
    assert PredictedKernel(legacy, 12.5).name == "k"


def test_flatten_kernels_modes():
    v100 = Device.V100
    full = [("smsp__sass_thread_inst_executed_ops_fadd_fmul_ffma_pred_on.avg.pct_of_peak_sustained_elapsed", 35.0),
            ("dram__bytes_read.sum", 3e8), ("dram__bytes_write.sum", 1e8)]
    a = KernelInstance("a", 100, 256, 1024, 512, 32, 1000, full)
    b = KernelInstance("b", 200, 64, 0, 0, 300, 2000)
    ks = [MeasuredKernel(a, [a], v100), MeasuredKernel(b, [], v100)]
    arrays, metrics, names = wave_batch.flatten_kernels(ks, wave_batch.UNIFIED)
    assert names == ["a", "b"] and list(arrays["smem_bytes"]) == [1536, 0]
    assert list(metrics["has_metrics"]) == [1, 0] and metrics["dram_read_bytes"][0] == 3e8
    assert arrays["regs_per_thread"][1] == 300
    _, none, _ = wave_batch.flatten_kernels(ks, wave_batch.RESIMPLIFIED)
    assert none is None
    with pytest.raises(AttributeError):
        wave_batch.flatten_kernels(ks, wave_batch.ROOFLINE)
    with pytest.raises(ZeroDivisionError):
        wave_batch.raise_like_reference(np.array([[1.5, np.nan]]))
    wave_batch.raise_like_reference(np.array([[1.5, 2.5]]))


def test_metadata_manager(tmp_path):
    path = str(tmp_path / "k.sqlite")
    con = sqlite3.connect(path)
    con.execute("CREATE TABLE kernels (name TEXT, arch INT, registers_per_thread INT)")
    con.executemany("INSERT INTO kernels VALUES (?, ?, ?)",
                    [("gemm", 61, 96), ("gemm", 70, 120), ("relu", 75, 16)])
    con.commit()
    con.close()
    m = MetadataManager(path)
    k = KernelInstance("gemm", 1, 32)
    assert m.kernel_registers_for(k, Device.V100) == 120
    assert m.kernel_registers_for(k, Device.P4000) == 96
    assert m.kernel_registers_for(k, Device.P100) is None            # arch 60 < 61
    assert m.kernel_registers_for(KernelInstance("other", 1, 32), Device.V100) is None
    mat = m.registers_matrix(["gemm", "relu", "x"], [Device.P100, Device.V100, Device.T4])
    assert mat.tolist() == [[-1, -1, -1], [120, -1, -1], [120, 16, -1]]
    assert MetadataManager(None).registers_matrix(["gemm"], [Device.V100]) is None
    assert len(m) == 3


def test_run_times_and_operations():
    dev = Device.V100
    ks = [PredictedKernel(None, 1.5e6), PredictedKernel(None, 0.5e6)]
    rt = RunTimePrediction(overhead_ns=1e6, predicted_kernels=ks, device=dev)
    assert rt.run_time_ms == 3.0 and rt.ktime_ns == 2e6 and rt.kernels is ks
    with pytest.raises(ValueError):
        RunTimePurePrediction(None, dev)
    fwd = RunTimeMeasurement(2.0, [], dev)
    op = MeasuredOperation("relu", Arguments((), {}), fwd, RunTimeMeasurement(1.0, [], dev), dev)
    assert op.run_time_ms == 3.0 and repr(op) == "relu" and op.to_device(dev, None) is op
    pred = PredictedOperation(op, RunTimePurePrediction(4.0, dev), None, dev)
    assert pred.run_time_ms == 4.0 and pred.name == "relu"
    with pytest.raises(RuntimeError):
        pred.to_device(dev, None)
    assert ns_to_ms(ms_to_ns(1.25)) == 1.25
    assert name_all_arguments(["a", "b"], (1,), {"b": 2, "c": 3}) == {"a": 1, "b": 2, "c": 3}
    assert {"conv2d", "gru"} <= SPECIAL_OPERATIONS


def test_thread_block_occupancy_known_answers(device_file):
    """KernelInstance.thread_block_occupancy is evaluated on the host by the library's own integer
    code: the known answers of the reference's calculator, without a GPU."""
    kat = [((256, 0, 0, 32), (8, 4, 8, 8)), ((1024, 0, 0, 65), (0, 0, 0, 0)),
           ((128, 16384, 0, 40), (6, 4, 4, 6)), ((64, 0, 49152, 16), (2, 1, 1, 2)),
           ((256, 8448, 0, 24), (8, 4, 7, 8)), ((96, 0, 40000, 72), (2, 1, 1, 2))]
    for (block, dyn, static, regs), expect in kat:
        k = KernelInstance("k", 100, block, dyn, static, regs, 1000)
        got = tuple(k.thread_block_occupancy(device_file[n]) for n in ("V100", "T4", "P100", "P4000"))
        assert got == expect
    k = KernelInstance("k", 100, 256, 0, 0, 64, 1000)
    assert k.thread_block_occupancy(device_file["V100"], 32) == 8


def test_feature_extraction():
    dev = Device.V100

    def op(name, args, kwargs=None, special=None):
        a = Arguments(args, kwargs or {})
        a.special.update(special or {})
        return MeasuredOperation(name, a, RunTimeMeasurement(1.0, [], dev), None, dev)

    conv = op("conv2d", ((32, 3, 224, 224), (64, 3, 7, 7), None, (2, 2), (3, 3), (1, 1), 1))
    assert conv2d_features(conv) == dict(batch=32, image_size=224, in_channels=3, out_channels=64,
                                         kernel_size=7, stride=2, padding=3, bias=0)
    conv_kw = op("conv2d", ((8, 16, 32, 32), (4, 16, 3, 3)), dict(bias=(4,), stride=1, padding=0))
    assert conv2d_features(conv_kw)["bias"] == 1 and conv2d_features(conv_kw)["stride"] == 1
    lin = op("linear", ((32, 50, 512), (1000, 512), (1000,)))
    assert linear_features(lin) == dict(batch=1600, in_features=512, out_features=1000, bias=1)
    assert bmm_features(op("bmm", ((8, 10, 20), (8, 20, 30)))) == dict(batch=8, left=10, middle=20, right=30)
    plain = op("lstm", ((35, 20, 650), ((2, 20, 650), (2, 20, 650)), [], True, 2, 0.5, True, False, False))
    assert lstm_features(plain) == dict(bias=1, bidirectional=0, batch=20, seq_len=35, input_size=650,
                                        hidden_size=650, num_layers=2)
    packed = op("lstm", ((700, 512), (20, 20, 18, 15), ((1, 20, 256),) * 2, [], True, 1, 0.0, True, True),
                special={"batch_sizes": [20, 20, 18, 15]})
    assert lstm_features(packed) == dict(bias=1, bidirectional=1, batch=20, seq_len=35, input_size=512,
                                         hidden_size=256, num_layers=1)

    # the batched extraction (positional fast path, named fall-back) agrees with the named one
    from habitat_b200.analysis.predictor import _EXTRACTORS, feature_matrix
    orders = {"conv2d": ["bias", "batch", "image_size", "in_channels", "out_channels", "kernel_size",
                         "stride", "padding"],
              "linear": ["bias", "batch", "in_features", "out_features"],
              "bmm": ["batch", "left", "middle", "right"],
              "lstm": ["bias", "bidirectional", "batch", "seq_len", "input_size", "hidden_size", "num_layers"]}
    groups = {"conv2d": [conv, conv, op("conv2d", ((1, 8, 9, 9), (16, 8, 5, 5), (16,), 1, 2, 1, 1))],
              "linear": [lin, op("linear", ((7, 512), (10, 512), None))],
              "bmm": [op("bmm", ((8, 10, 20), (8, 20, 30), None)), op("bmm", ((2, 3, 4), (2, 4, 5)))],
              "lstm": [plain, packed]}
    for name, ops in groups.items():
        want = np.array([[_EXTRACTORS[name](o)[f] for f in orders[name]] for o in ops], np.float32)
        assert np.array_equal(feature_matrix(name, ops, orders[name]), want), name
    mixed = [conv, conv_kw]                      # one keyword recording sends the group down the named path
    want = np.array([[conv2d_features(o)[f] for f in orders["conv2d"]] for o in mixed], np.float32)
    assert np.array_equal(feature_matrix("conv2d", mixed, orders["conv2d"]), want)


def test_runtime_predictor_checkpoints(tmp_path):
    import torch
    torch.manual_seed(3)
    p = RuntimePredictor("bmm", 2, 1024)
    assert p.model.features == ["batch", "left", "middle", "right"]
    assert p.device_params == ["mem", "mem_bw", "num_sm", "single"]
    p.mu, p.sigma = np.arange(8.0), np.arange(8.0) + 1
    path = str(tmp_path / "model.pth")
    p.save_state(path)
    keys = set(torch.load(path, weights_only=False)["model"])
    assert {"fc1.weight", "mlp.layers.0.weight", "mlp.layers.2.bias", "fc2.bias"} <= keys
    q = RuntimePredictor("bmm", 2, 1024, path)
    assert np.array_equal(q.mu, p.mu) and torch.equal(q.model.fc1.weight, p.model.fc1.weight)
    assert get_device_features("V100", ["mem", "single"]) == [16.0, 14.028]
    assert set(workloads.BENCH_DEVICES) <= set(get_all_devices(["mem"]))
    with pytest.raises(IndexError):
        get_device_features("NoSuchGPU", ["mem"])


def test_workloads_are_seeded():
    a, b = workloads.make_kernels(100, 5), workloads.make_kernels(100, 5)
    assert all(np.array_equal(a[k], b[k]) for k in a)
    assert a["num_blocks"].min() >= 1 and a["num_blocks"].max() <= 1 << 20
    assert set(np.unique(a["block_size"])) <= {32, 64, 128, 256, 512, 1024}
    assert a["smem_bytes"].max() <= 96 * 1024 and (a["smem_bytes"] % 256 == 0).all()
    f, d = workloads.make_queries("lstm", 50, 1)
    assert f.shape == (50, 7) and d.max() < 6 and f[:, 4].min() >= 32
    mu, sigma = workloads.batch_mu_sigma(f, d)
    assert mu.shape == (11,) and (sigma > 0).all()


def test_precision_knob(monkeypatch):
    from habitat_b200.analysis.predictor import Predictor
    assert Predictor()._precision == "bf16"
    monkeypatch.setenv("HABITAT_B200_PRECISION", "bf16x3")
    assert Predictor()._precision == "bf16x3"
    assert Predictor(precision="bf16")._precision == "bf16"
    monkeypatch.setenv("HABITAT_B200_PRECISION", "fp64")
    with pytest.raises(ValueError):
        Predictor()
