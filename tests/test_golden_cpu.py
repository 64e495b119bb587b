"""The CPU oracle against fixtures produced by the reference's own Python code.

These are what pins the oracle's scaling formulas and MLP forward: the reference
has no tests or golden vectors of its own, so tests/golden/make_golden.py ran
its wave_scaling/*.py and RuntimePredictor.predict on seeded inputs.
"""
import numpy as np
import pytest

from oracle import mlp as omlp
from oracle import wave as owave
from tests import golden_util as gu


def _expected(strategy, has_metrics, gamma_fn):
    """gamma the oracle must use to reproduce `strategy` for one kernel."""
    if strategy == "resimplified":
        return 1.0
    if not has_metrics:
        return None if strategy == "roofline" else 1.0
    return gamma_fn()


@pytest.mark.parametrize("strategy", ["roofline", "resimplified", "unified"])
def test_wave_scaling_formulas(device_file, strategy):
    g = gu.load("wave_scaling.npz")
    names = [str(n) for n in g["device_names"]]
    devs = [device_file[n] for n in names]
    kernel_names = [str(n) for n in g["kernel_names"]]
    rows = [tuple(r) for r in g["metadata_rows"]]
    want = g[strategy]
    K = len(g["num_blocks"])
    checked = raised = 0
    for o, origin in enumerate(devs):
        for d, dest in enumerate(devs):
            arch = gu.arch_of(dest)
            for k in range(K):
                smem = int(g["dynamic_smem"][k]) + int(g["static_smem"][k])
                gamma = _expected(strategy, bool(g["has_metrics"][k]), lambda: owave.roofline_gamma(
                    g["flop_efficiency"][k], g["dram_read"][k], g["dram_write"][k], g["run_time_ns"][k],
                    origin.spec_tuple(), dest.spec_tuple()))
                if gamma is None:
                    assert np.isnan(want[o, d, k])      # roofline needs metrics (AttributeError)
                    continue
                dest_regs = gu.metadata_lookup(rows, kernel_names[g["kernel_name_index"][k]], arch)
                st, ns, oo, od = owave.wave_scale_pair(
                    origin.spec_tuple(), dest.spec_tuple(), g["num_blocks"][k], g["block_size"][k],
                    smem, g["regs"][k], dest_regs, g["run_time_ns"][k], gamma)
                assert oo == g["occupancy"][o, k]
                if np.isnan(want[o, d, k]):
                    assert st >= 2, (o, d, k)
                    raised += 1
                else:
                    assert st <= 1, (o, d, k)
                    assert abs(ns - want[o, d, k]) <= 1e-12 * want[o, d, k], (o, d, k)
                    checked += 1
    assert checked > 2000 and raised > 100


def test_scaling_known_answers(device_file):
    """V100 -> T4 values read off the reference (metrics 35 %, 3e8 B read, 1e8 B written)."""
    v100, t4 = device_file["V100"].spec_tuple(), device_file["T4"].spec_tuple()
    gamma = owave.roofline_gamma(35.0, 3e8, 1e8, 1_000_000, v100, t4)
    assert abs(gamma - 0.582025311788275) < 1e-15
    st, ns, _, _ = owave.wave_scale_pair(v100, t4, 10000, 256, 0, 32, -1, 1_000_000, gamma)
    assert st == 0 and abs(ns - 3612227.7495064945) < 1e-6
    gamma = owave.roofline_gamma(35.0, 3e8, 1e8, 50_000, v100, t4)
    st, ns, _, _ = owave.wave_scale_pair(v100, t4, 100, 256, 0, 32, -1, 50_000, gamma)
    assert st == 1 and abs(ns - 51283.88343614581) < 1e-8
    st, ns, _, _ = owave.wave_scale_pair(v100, t4, 10000, 256, 0, 32, -1, 1_000_000, 1.0)
    assert abs(ns - 3092050.2092050207) < 1e-6


@pytest.mark.parametrize("op", ["linear", "lstm", "conv2d", "bmm"])
def test_mlp_forward(op):
    """oracle/mlp.py against RuntimePredictor.predict of the reference, query by query."""
    from habitat_b200 import workloads
    from habitat_b200.analysis.mlp.devices import get_device_features
    g = gu.load("mlp_predict.npz")
    w = workloads.torch_init_mlp_weights(op, seed=int(g[op + "_weight_seed"]))
    names = [str(n) for n in g[op + "_device"]]
    uniq = sorted(set(names))
    table = np.array([get_device_features(n, ["mem", "mem_bw", "num_sm", "single"]) for n in uniq])
    rows = np.array([uniq.index(n) for n in names])
    got = omlp.predict(w, g[op + "_features"], rows, table, g[op + "_mu"], g[op + "_sigma"])
    want = g[op + "_prediction"]
    assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max()
