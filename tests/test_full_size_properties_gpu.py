"""Full benchmark sizes, checked through properties that need no CPU reference at scale.

The scale-sweep configuration has 11,184,811 kernels x 6 devices and 4,194,304 queries
per predictor; the oracle would take minutes there, so it only sees a strided subset,
and the rest is covered by exact algebraic properties of the path.
"""
import numpy as np
import pytest
import torch

from habitat_b200 import batched, workloads
from tests.helpers import run_wave_oracle, to_numpy

pytestmark = pytest.mark.gpu

K_FULL = 11_184_812          # 67,108,864 pairs / 6, padded to a multiple of 4


def test_wave_scaling_full_size(bench_devices):
    kernels = workloads.make_kernels(K_FULL, seed=1005)
    kb = batched.KernelBatch.from_numpy(kernels)
    origin = bench_devices[0]
    res = batched.wave_scale(kb, origin, bench_devices)
    ns = res.scaled_ns

    # 1. the origin listed as a destination: every valid pair keeps its time, bit for bit
    t = kb.run_time_ns
    valid = ~torch.isnan(ns[0])
    assert torch.equal(ns[0][valid], t[valid])
    assert torch.equal(res.dest_occupancy[0], res.origin_occupancy)
    assert torch.equal(res.dest_waves[0], res.origin_waves)
    # V100_32 has the same scaling fields (NaN where the reference raises, on both)
    assert torch.equal(torch.nan_to_num(ns[1], nan=-1.0), torch.nan_to_num(ns[0], nan=-1.0))

    # 2. linear in the measured time: doubling t doubles every prediction exactly
    kb2 = batched.KernelBatch(kb.num_blocks, kb.block_size, kb.regs_per_thread, kb.smem_bytes,
                              kb.run_time_ns * 2, kb.gamma)
    res2 = batched.wave_scale(kb2, origin, bench_devices)
    assert torch.equal(torch.nan_to_num(res2.scaled_ns, nan=-1.0), torch.nan_to_num(ns * 2, nan=-1.0))
    assert torch.equal(res2.dest_occupancy, res.dest_occupancy)

    # 3. NaN exactly where a wave size the reference divides by is zero
    occ_o = res.origin_occupancy.to(torch.int32)
    nb = kb.num_blocks
    for d, dev in enumerate(bench_devices):
        occ_d = res.dest_occupancy[d].to(torch.int32)
        small_o = nb < occ_o * origin.num_sms
        raises = (occ_o == 0) | (small_o & (occ_d == 0))
        assert torch.equal(torch.isnan(ns[d]), raises)
        # occupancy never exceeds the blocks-per-SM limit; waves consistent with occupancy
        assert int(occ_d.max()) <= 32
        w = res.dest_waves[d].view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        ok = occ_d > 0
        wave = (occ_d * dev.num_sms).to(torch.int64)
        assert torch.equal(w[ok], (nb.to(torch.int64)[ok] // wave[ok]))
        assert bool((w[~ok] == 0xFFFFFFFF).all())

    # 4. gamma = 1 makes every large-kernel factor the bandwidth ratio (resimplified rule)
    kb1 = batched.KernelBatch(kb.num_blocks, kb.block_size, kb.regs_per_thread, kb.smem_bytes,
                              kb.run_time_ns, torch.ones_like(kb.gamma))
    r1 = batched.wave_scale(kb1, origin, bench_devices, want_status=True)
    for d, dev in enumerate(bench_devices):
        large = r1.status[d] == 0
        ratio = (r1.scaled_ns[d][large] / kb.run_time_ns[large]).double()
        want = origin.mem_bandwidth_gb / dev.mem_bandwidth_gb
        assert float((ratio / want - 1).abs().max()) <= 1e-6
        small = r1.status[d] == 1
        assert torch.equal(r1.scaled_ns[d][small], kb.run_time_ns[small])

    # 5. a strided 1/64 subset against the oracle
    idx = np.arange(0, K_FULL, 64)
    sub = {k: v[idx] for k, v in kernels.items()}
    ref = run_wave_oracle(sub, origin, bench_devices)
    got = to_numpy(ns)[:, idx]
    okm = ref["status"] <= 1
    assert np.array_equal(np.isnan(got), ~okm)
    err = np.abs(got[okm] - ref["scaled_ns"][okm]) / ref["scaled_ns"][okm]
    assert err.max() <= 1e-6
    assert np.array_equal(to_numpy(res.dest_occupancy)[:, idx], ref["dest_occupancy"])
    assert np.array_equal(to_numpy(res.dest_waves)[:, idx], ref["dest_waves"])

    # 6. per-destination totals: the device reduction equals a float64 sum of the plane
    totals = batched.plane_sum(ns).cpu().numpy()
    want = np.nansum(to_numpy(ns).astype(np.float64), axis=1)
    assert np.allclose(totals, want, rtol=1e-12)


@pytest.mark.parametrize("op", ["conv2d", "lstm"])
def test_mlp_full_size(op):
    Q = 4_194_304
    w = workloads.torch_init_mlp_weights(op)
    feats, dev = workloads.make_queries(op, Q, 1005)
    mu, sigma = workloads.batch_mu_sigma(feats, dev)
    h = batched.MLPHandle(feats.shape[1], mu=mu, sigma=sigma,
                          device_features=workloads.BENCH_DEVICE_FEATURES, **w)
    f, r = torch.from_numpy(feats).cuda(), torch.from_numpy(dev).cuda()
    out = h.predict(f, r)
    # a prediction depends on its own query only: any sub-batch reproduces it bit for bit
    for lo, n in ((0, 4096), (1_000_003, 777), (Q - 130, 130)):
        part = h.predict(f[lo:lo + n].contiguous(), r[lo:lo + n].contiguous())
        assert torch.equal(part, out[lo:lo + n])
    # duplicated queries give identical answers wherever they sit in a tile
    perm = torch.randperm(8192, device="cuda")
    a = h.predict(f[:8192][perm].contiguous(), r[:8192][perm].contiguous())
    assert torch.equal(a, out[:8192][perm])
    h.check_status()
    # strided subset against the float32 oracle
    from oracle import mlp as omlp
    idx = np.arange(0, Q, 1024)
    ref = omlp.predict(w, feats[idx], dev[idx], workloads.BENCH_DEVICE_FEATURES, mu, sigma)
    got = out.cpu().numpy()[idx]
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref)).all()
    assert np.isfinite(out.cpu().numpy()).all()
    h.close()


def test_config1_split_precision_full_size():
    """65,536 linear queries on the hi/lo split path: 1e-4 against the float32 reference."""
    from oracle import mlp as omlp
    op, Q = "linear", 65536
    w = workloads.torch_init_mlp_weights(op)
    feats, dev = workloads.make_queries(op, Q, 1001)
    mu, sigma = workloads.batch_mu_sigma(feats, dev)
    h = batched.MLPHandle(4, mu=mu, sigma=sigma, device_features=workloads.BENCH_DEVICE_FEATURES,
                          precision="bf16x3", **w)
    f, r = torch.from_numpy(feats).cuda(), torch.from_numpy(dev).cuda()
    h.predict(f, r)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    out = h.predict(f, r)
    e1.record()
    torch.cuda.synchronize()
    h.check_status()
    ref = omlp.predict(w, feats, dev, workloads.BENCH_DEVICE_FEATURES, mu, sigma)
    got = out.cpu().numpy()
    assert (np.abs(got - ref) <= 1e-4 * np.abs(ref)).all()
    print("config 1: %d queries in %.2f ms (split precision), max rel err %.2g"
          % (Q, e0.elapsed_time(e1), (np.abs(got - ref) / np.abs(ref)).max()))
    h.close()
