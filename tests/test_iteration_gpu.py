"""Mixed iteration traces: per-iteration totals on the device against the oracle.

The shape of one iteration follows the benchmark's mixed trace: 53 conv2d, 1 linear
and 32 bmm operations predicted by their MLPs plus 74 ordinary operations of one
wave-scaled kernel each; totals within 2e-2 relative of the float64 reference.
"""
import numpy as np
import pytest
import torch

from habitat_b200 import batched, iteration, workloads
from oracle import mlp as omlp
from oracle import wave as owave

pytestmark = pytest.mark.gpu

PER_ITER = {"conv2d": 53, "linear": 1, "bmm": 32}
KERNELS_PER_ITER = 74


def _make(I, seed, origin_spec):
    def occ(block, smem, regs):
        return np.array([owave.occupancy(origin_spec, b, s, r)[0] for b, s, r in zip(block, smem, regs)])
    kernels = workloads.make_kernels(I * KERNELS_PER_ITER, seed, valid_only=True, origin=occ)
    g = workloads.rng(seed + 1)
    overhead = g.uniform(0, 10_000, size=I * KERNELS_PER_ITER).astype(np.float32)      # ns
    ops = {}
    for op, n in PER_ITER.items():
        feats, _ = workloads.make_queries(op, I * n, seed + 7 + len(op))
        rt = np.exp(g.uniform(np.log(0.02), np.log(50.0), size=I * n)).astype(np.float32)
        ops[op] = (feats, rt)
    return kernels, overhead, ops


@pytest.mark.parametrize("I", [3, 64, 512])
def test_iteration_totals(bench_devices, I):
    origin, dests = bench_devices[0], bench_devices
    kernels, overhead, ops = _make(I, 4004, origin.spec_tuple())
    koff = np.arange(I + 1, dtype=np.int64) * KERNELS_PER_ITER
    devf = workloads.BENCH_DEVICE_FEATURES

    special, weights, stats = {}, {}, {}
    for op, (feats, rt) in ops.items():
        w = workloads.torch_init_mlp_weights(op)
        dev_all = np.tile(np.arange(6, dtype=np.uint8), len(feats))[:len(feats)]
        mu, sigma = workloads.batch_mu_sigma(feats, dev_all)
        weights[op], stats[op] = w, (mu, sigma)
        h = batched.MLPHandle(feats.shape[1], mu=mu, sigma=sigma, device_features=devf, **w)
        off = torch.from_numpy(np.arange(I + 1, dtype=np.int64) * PER_ITER[op]).cuda()
        special[op] = iteration.SpecialOps(h, torch.from_numpy(feats).cuda(), torch.from_numpy(rt).cuda(), off)

    totals, wave = iteration.predict_iteration_totals(
        batched.KernelBatch.from_numpy(kernels), torch.from_numpy(overhead).cuda(),
        torch.from_numpy(koff).cuda(), special, origin, dests, 0, list(range(6)))
    torch.cuda.synchronize()
    for s in special.values():
        s.handle.check_status()
    got = totals.cpu().numpy()
    assert not torch.isnan(wave.scaled_ns).any()       # valid-only kernels never raise
    assert batched.wave_scale_path() == "wave_scale_lut_kernel"

    # reference: the oracle, float64, operation by operation
    specs = [d.spec_tuple() for d in dests]
    ref = owave.wave_scale_batch(specs, 0, list(range(6)), kernels, want_limits=False)
    want = np.zeros((I, 6))
    for d in range(6):
        ns = kernels["run_time_ns"] if d == 0 else ref["scaled_ns"][d]     # row 0 is the origin itself
        want[:, d] = (overhead.astype(np.float64) + ns).reshape(I, -1).sum(axis=1) / 1e6
    for op, (feats, rt) in ops.items():
        mu, sigma = stats[op]
        n = len(feats)
        p_orig = omlp.predict(weights[op], feats, np.zeros(n, np.uint8), devf, mu, sigma, np.float64)
        for d in range(6):
            if d == 0:
                ms = rt.astype(np.float64)
            else:
                p_dest = omlp.predict(weights[op], feats, np.full(n, d, np.uint8), devf, mu, sigma, np.float64)
                ms = np.maximum(rt.astype(np.float64) * p_dest / p_orig, 0)
            want[:, d] += ms.reshape(I, -1).sum(axis=1)
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).min()
    assert np.abs(got[:, 0] - want[:, 0]).max() <= 1e-6 * want[:, 0].max()   # identity column
    print("config-4 style totals, max rel err %.3g" % (np.abs(got - want) / want).max())
