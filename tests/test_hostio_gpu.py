"""Host pipelines (one pinned block in, pinned results out, three streams) against the device entry points."""
import numpy as np
import pytest
import torch

from habitat_b200 import batched, hostio, workloads
from tests.helpers import run_wave_oracle, to_numpy

pytestmark = pytest.mark.gpu


def test_wave_scale_pipeline(bench_devices):
    K = 40000
    batches = [workloads.make_kernels(K, seed=300 + i) for i in range(5)]
    every = ("scaled_ns", "dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves")
    pipe = hostio.WaveScaleHost(bench_devices[0], bench_devices, K, depth=3, results=every)
    blocks = [hostio.pack_kernels(b) for b in batches]
    assert blocks[0].is_pinned() and blocks[0].numel() == 20 * K
    for i, b in enumerate(batches):
        slot = i % 3
        pipe.wait(slot)                      # results of batch i - 3 were consumed below
        pipe.submit(blocks[i], slot)
        if i >= 1:                           # check the previous batch while this one runs
            prev = (i - 1) % 3
            pipe.wait(prev)
            ref = run_wave_oracle(batches[i - 1], bench_devices[0], bench_devices)
            got = {k: to_numpy(v) for k, v in pipe.host_out[prev].items()}
            for key in ("dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves"):
                assert np.array_equal(got[key], ref[key])
            ok = ref["status"] <= 1
            assert np.isnan(got["scaled_ns"][~ok]).all()
            err = np.abs(got["scaled_ns"][ok] - ref["scaled_ns"][ok]) / ref["scaled_ns"][ok]
            assert err.max() <= 1e-6
    assert pipe.h2d_bytes == 20 * K and pipe.d2h_bytes == (9 * 6 + 5) * K

    # only the predicted times copied back; the other outputs stay on the device
    times = hostio.WaveScaleHost(bench_devices[0], bench_devices, K, depth=2, results=("scaled_ns",))
    times.submit(blocks[0], 0)
    times.wait(0)
    ref = run_wave_oracle(batches[0], bench_devices[0], bench_devices)
    ok = ref["status"] <= 1
    got = to_numpy(times.host_out[0]["scaled_ns"])
    assert list(times.host_out[0]) == ["scaled_ns"] and times.d2h_bytes == 4 * 6 * K
    assert np.isnan(got[~ok]).all() and (np.abs(got[ok] - ref["scaled_ns"][ok]) <= 1e-6 * ref["scaled_ns"][ok]).all()
    assert np.array_equal(to_numpy(times.dev_out[0].dest_occupancy), ref["dest_occupancy"])
    # totals only: the per-destination sums of a batch come back, nothing else is downloaded
    sums = hostio.WaveScaleHost(bench_devices[0], bench_devices, K, depth=2, results=("totals",))
    for i in range(3):
        sums.wait(i % 2)
        sums.submit(blocks[i], i % 2)
    sums.wait(0)
    ref2 = run_wave_oracle(batches[2], bench_devices[0], bench_devices)
    want = np.where(ref2["status"] <= 1, ref2["scaled_ns"], 0.0).sum(axis=1)
    assert list(sums.host_out[0]) == ["totals"] and sums.d2h_bytes == 8 * 6
    np.testing.assert_allclose(to_numpy(sums.host_out[0]["totals"]), want, rtol=1e-6)
    np.testing.assert_allclose(to_numpy(sums.host_out[0]["totals"]),
                               np.nansum(to_numpy(sums.dev_out[0].scaled_ns).astype(np.float64), axis=1), rtol=1e-13)
    with pytest.raises(ValueError):
        hostio.WaveScaleHost(bench_devices[0], bench_devices, K, results=("scaled",))
    with pytest.raises(ValueError):
        times.submit(blocks[0][:-20], 1)
    # pinned pages are placed near the GPU when the topology can be read; either way the
    # thread's CPU set is what it was afterwards
    import os
    before = os.sched_getaffinity(0)
    with hostio.numa_local(torch.cuda.current_device()) as cpus:
        assert cpus is None or cpus <= before
    assert os.sched_getaffinity(0) == before


def test_mlp_pipeline():
    op, Q = "linear", 5000
    w = workloads.torch_init_mlp_weights(op)
    feats, dev = workloads.make_queries(op, Q, 17)
    mu, sigma = workloads.batch_mu_sigma(feats, dev)
    h = batched.MLPHandle(4, mu=mu, sigma=sigma, device_features=workloads.BENCH_DEVICE_FEATURES, **w)
    want = h.predict(torch.from_numpy(feats).cuda(), torch.from_numpy(dev).cuda()).cpu()
    pipe = hostio.MLPPredictHost(4, Q + 100, depth=2)          # buffers may be larger than a batch
    pf, pr = torch.from_numpy(feats).pin_memory(), torch.from_numpy(dev).pin_memory()
    for i in range(4):
        pipe.wait(i % 2)
        pipe.submit(h, pf, pr, i % 2)
    for slot in range(2):
        pipe.wait(slot)
        assert torch.equal(pipe.host_out[slot][:Q], want)
    h.check_status()
    h.close()
