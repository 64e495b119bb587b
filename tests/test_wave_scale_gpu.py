"""Wave scaling on the GPU (through the C ABI) against the C oracle."""
import numpy as np
import pytest
import torch

from habitat_b200 import batched, workloads
from oracle import wave as owave
from tests.helpers import assert_wave_equal, run_wave_gpu, run_wave_oracle, to_numpy

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K", [1, 3, 4, 31, 32, 33, 1025, 4096, 65536 + 4])
@pytest.mark.parametrize("D", [1, 6])
def test_sizes_and_tails(bench_devices, K, D):
    kernels = workloads.make_kernels(K, seed=K * 7 + D)
    origin, dests = bench_devices[0], bench_devices[:D] if D > 1 else [bench_devices[5]]
    assert_wave_equal(run_wave_gpu(kernels, origin, dests), run_wave_oracle(kernels, origin, dests))


def test_empty_batch(bench_devices):
    kernels = workloads.make_kernels(0, seed=1)
    res = run_wave_gpu(kernels, bench_devices[0], bench_devices)
    assert res["scaled_ns"].shape == (6, 0)


def test_config2_full(bench_devices):
    """1,048,576 kernels to the six benchmark rows."""
    kernels = workloads.make_kernels(1 << 20, seed=1002)
    got = run_wave_gpu(kernels, bench_devices[0], bench_devices)
    ref = run_wave_oracle(kernels, bench_devices[0], bench_devices)
    worst = assert_wave_equal(got, ref)
    frac_err = (ref["status"] >= 2).mean()
    assert 0.5 < frac_err < 0.7          # most draws cannot run on the origin at all
    print("config 2: max rel err %.3g, %.1f%% pairs raise in the reference" % (worst, 100 * frac_err))


def test_valid_only_and_all_device_rows(device_file):
    names = sorted(device_file)
    devs = [device_file[n] for n in names]
    origin = device_file["V100"]
    spec = origin.spec_tuple()

    def occ(block, smem, regs):
        return np.array([owave.occupancy(spec, b, s, r)[0] for b, s, r in zip(block, smem, regs)])

    kernels = workloads.make_kernels(20000, seed=5, valid_only=True, origin=occ)
    got = run_wave_gpu(kernels, origin, devs)
    ref = run_wave_oracle(kernels, origin, devs)
    assert_wave_equal(got, ref)
    assert (ref["origin_occupancy"] > 0).all()


def test_every_origin(device_file):
    devs = [device_file[n] for n in sorted(device_file)]
    kernels = workloads.make_kernels(3000, seed=9)
    kernels["regs_per_thread"][:64] = np.arange(0, 64 * 5, 5).astype(np.uint16)   # incl. 0 and > 256
    kernels["block_size"][64:128] = np.arange(1, 1100, 17)[:64].astype(np.uint16)
    kernels["smem_bytes"][128:160] = np.linspace(0, 240 * 1024, 32).astype(np.uint32)
    kernels["smem_bytes"][160] = 0xFFFFFFFF
    kernels["block_size"][161] = 0
    kernels["num_blocks"][162] = 0
    kernels["num_blocks"][163] = -5
    for origin in devs:
        assert_wave_equal(run_wave_gpu(kernels, origin, devs), run_wave_oracle(kernels, origin, devs))


def test_dest_regs(bench_devices):
    K = 5000
    kernels = workloads.make_kernels(K, seed=12)
    g = workloads.rng(13)
    dest_regs = g.integers(-1, 256, size=(6, K)).astype(np.int16)
    dest_regs[:, ::3] = -1
    got = run_wave_gpu(kernels, bench_devices[0], bench_devices, dest_regs=dest_regs)
    ref = run_wave_oracle(kernels, bench_devices[0], bench_devices, dest_regs=dest_regs)
    assert_wave_equal(got, ref)
    # register overrides and the status plane are served by the tabulated kernel
    assert got["fast_path"] == "wave_scale_lut_kernel" and got["plain_path"] == "wave_scale_lut_kernel"
    odd = {k: v[:K - 1] for k, v in kernels.items()}          # odd K: one record per thread
    got = run_wave_gpu(odd, bench_devices[0], bench_devices, dest_regs=dest_regs[:, :K - 1])
    assert got["fast_path"] == "wave_scale_lut_kernel"
    assert_wave_equal(got, run_wave_oracle(odd, bench_devices[0], bench_devices, dest_regs=dest_regs[:, :K - 1]))


def test_metrics_mode(device_file):
    """gamma from raw metrics, per (kernel, destination) pair."""
    K = 8192
    devs = [device_file[n] for n in ("T4", "V100", "P100", "B200", "A100_40")]
    origin = device_file["V100"]
    kernels = workloads.make_kernels(K, seed=21)
    metrics = workloads.make_metrics(K, seed=22)
    got = run_wave_gpu(kernels, origin, devs, metrics=metrics)
    # gamma from raw metrics is computed inside the tabulated kernel (six rows with more than
    # four shared-memory classes: every row's own tables)
    assert got["fast_path"] == "wave_scale_lut_kernel" and got["plain_path"] == "wave_scale_lut_kernel"
    for d, dest in enumerate(devs):
        gam = np.array([
            owave.roofline_gamma(metrics["flop_efficiency_pct"][k], metrics["dram_read_bytes"][k],
                                 metrics["dram_write_bytes"][k], kernels["run_time_ns"][k],
                                 origin.spec_tuple(), dest.spec_tuple())
            if metrics["has_metrics"][k] else 1.0 for k in range(K)])
        assert ((gam >= 0) & (gam <= 1)).all()
        k2 = dict(kernels, gamma=gam.astype(np.float32))
        ref = run_wave_oracle(k2, origin, [dest])
        one = {k: (v[d:d + 1] if k not in ("origin_occupancy", "origin_waves", "limits") else v)
               for k, v in got.items() if isinstance(v, np.ndarray)}
        one["limits"] = got["limits"][[0, d + 1]]
        for name in ("fast", "plain"):
            one[name] = {k: (v[d:d + 1] if k not in ("origin_occupancy", "origin_waves") else v)
                         for k, v in got[name].items()}
        # gamma reaches the oracle rounded to float32; the device keeps float64
        assert_wave_equal(one, ref, rel=2e-6)


def test_host_buffer_entry_point(bench_devices):
    kernels = workloads.make_kernels(10001, seed=31)
    res = batched.wave_scale_host(kernels, bench_devices[0], bench_devices, want_status=True,
                                  want_limits=True)
    assert_wave_equal(res, run_wave_oracle(kernels, bench_devices[0], bench_devices))


def test_reductions():
    g = workloads.rng(41)
    vals = g.uniform(0, 50, size=100000).astype(np.float32)
    cuts = np.sort(g.choice(100001, size=511, replace=False))
    offsets = np.concatenate([[0], cuts, [100000]]).astype(np.int64)
    got = batched.segment_sum(torch.from_numpy(vals).cuda(), torch.from_numpy(offsets).cuda()).cpu().numpy()
    ref = np.array([vals[a:b].astype(np.float64).sum() for a, b in zip(offsets[:-1], offsets[1:])])
    assert np.allclose(got, ref, rtol=1e-12, atol=1e-9)
    planes = g.uniform(0, 1e6, size=(6, 50001)).astype(np.float32)
    planes[:, ::7] = np.nan
    got = batched.plane_sum(torch.from_numpy(planes).cuda()).cpu().numpy()
    assert np.allclose(got, np.nansum(planes.astype(np.float64), axis=1), rtol=1e-12)
    # sums grouped by a key per element (per-device totals of MLP predictions), more than eight groups too
    for n_groups in (1, 6, 8, 9, 20):
        keys = g.integers(0, n_groups + 2, size=vals.size).astype(np.uint8)      # some keys beyond the groups
        v = vals.copy()
        v[::11] = np.nan
        got = batched.group_sum(torch.from_numpy(v).cuda(), torch.from_numpy(keys).cuda(), n_groups).cpu().numpy()
        ref = np.array([np.nansum(v[keys == k].astype(np.float64)) for k in range(n_groups)])
        assert np.allclose(got, ref, rtol=1e-12, atol=1e-9), n_groups
    rt = g.uniform(0.02, 50, 1000).astype(np.float32)
    pd = g.normal(1, 1, 1000).astype(np.float32)
    po = g.uniform(0.5, 2, 1000).astype(np.float32)
    cnt = torch.zeros(1, dtype=torch.int32, device="cuda").view(torch.uint32)
    got = batched.special_scale(torch.from_numpy(rt).cuda(), torch.from_numpy(pd).cuda(),
                                torch.from_numpy(po).cuda(), cnt).cpu().numpy()
    ref = np.maximum(rt.astype(np.float64) * pd / po, 0).astype(np.float32)
    assert np.array_equal(got, ref)
    assert int(cnt.view(torch.int32).cpu()[0]) == int((rt.astype(np.float64) * pd / po < 0).sum())


def _edge_records(devices):
    """Records on and around every boundary the tabulated limits are indexed by."""
    g = np.random.default_rng(77)
    blocks, block_size, regs, smem = [], [], [], []

    def add(nb, bs, rg, sm):
        blocks.append(nb); block_size.append(bs); regs.append(rg); smem.append(sm)

    for bs in list(range(0, 1100)) + [2048, 4096, 65535]:             # every warps-per-block step and beyond
        add(int(g.integers(1, 5000)), bs, int(g.integers(0, 300)), int(g.integers(0, 100_000)))
    for rg in list(range(0, 330)) + [512, 1000, 65535]:                # every register step, above 256 too
        add(int(g.integers(1, 5000)), int(g.choice([32, 96, 128, 256, 1000, 1024])), rg, int(g.integers(0, 60_000)))
    for sm in range(0, 262_400, 61):                                   # odd offsets across every 128-byte step
        add(int(g.integers(1, 5000)), int(g.choice([64, 256, 1024])), int(g.integers(0, 128)), sm)
    for step in range(0, 2060, 7):                                     # exactly on, below and above step edges
        for delta in (-1, 0, 1):
            add(77, 128, 32, max(0, step * 128 + delta))
    for sm in (0xFFFFFFFF, 0x80000000, 0x7FFF0001, 0x7FFF0000, 262_143, 262_144, 262_145):
        add(5, 128, 32, sm)
    # grid sizes around the wave sizes (SMs x occupancy) of every row, and the extremes
    for dev in devices:
        for occ in (1, 2, 3, 8, 16, 32):
            wave = dev.num_sms * occ
            for nb in (wave - 1, wave, wave + 1, 2 * wave - 1, 2 * wave, dev.num_sms - 1, dev.num_sms, dev.num_sms + 1):
                add(nb, int(g.choice([32, 64, 128, 256, 512, 1024])), int(g.integers(16, 128)),
                    int(g.integers(0, 48 * 1024)))
    for nb in (0, -1, -5, 1, 2, 2**31 - 1, 2**31 - 2, 2**30, 2**30 + 12345, 29_000_000, 29_100_000, 123_456_789):
        for bs in (32, 256, 1024):
            add(nb, bs, 32, 1024)
    n = len(blocks) + (len(blocks) & 1)                                # the tabulated kernel takes even K
    while len(blocks) < n:
        add(1, 32, 16, 0)
    return dict(
        num_blocks=np.array(blocks, np.int64).astype(np.int32),
        block_size=np.array(block_size, np.uint16), regs_per_thread=np.array(regs, np.uint16),
        smem_bytes=np.array(smem, np.uint64).astype(np.uint32),
        run_time_ns=np.exp(g.uniform(np.log(2e3), np.log(5e7), size=n)).astype(np.float64),
        gamma=g.uniform(0.0, 1.0, size=n).astype(np.float32))


def test_tabulated_kernel_on_edges(bench_devices, device_file):
    """The table kernel (taken for even K when every row qualifies) against the oracle on records
    that sit on, just below and just above every index boundary of its tables."""
    kernels = _edge_records(bench_devices)
    for origin in bench_devices:
        got = run_wave_gpu(kernels, origin, bench_devices)
        assert got["fast_path"] == "wave_scale_lut_kernel"
        assert_wave_equal(got, run_wave_oracle(kernels, origin, bench_devices))
    # other rows of the device file, in groups small enough to stay within four classes per limit
    names = sorted(device_file)
    taken = 0
    for i in range(0, len(names) - 2, 3):
        devs = [device_file[n] for n in names[i:i + 3]]
        got = run_wave_gpu(kernels, devs[0], devs)
        taken += got["fast_path"] == "wave_scale_lut_kernel"
        assert_wave_equal(got, run_wave_oracle(kernels, devs[0], devs))
    assert taken >= 2


@pytest.mark.parametrize("D", [33, 64])
def test_many_destinations(device_file, D):
    """More than 32 destinations per call take the generic kernel (the faster ones hold at most 32
    rows in their parameters); same results."""
    names = sorted(device_file)
    dests = [device_file[names[i % len(names)]] for i in range(D)]
    kernels = workloads.make_kernels(2000, seed=5)
    got = run_wave_gpu(kernels, device_file["V100"], dests)
    assert got["fast_path"] == "wave_scale_kernel"
    assert_wave_equal(got, run_wave_oracle(kernels, device_file["V100"], dests))


def _wave_with_partials(kernels, origin, dests, dest_regs=None, partials=None):
    kb = batched.KernelBatch.from_numpy(kernels)
    K, D = len(kb), len(dests)
    partials = partials or batched.WavePartials(K, D)
    out = batched.wave_scale(kb, origin, dests, dest_regs=dest_regs, partials=partials)
    path = batched.wave_scale_path()
    totals = partials.totals()
    torch.cuda.synchronize()
    return out, totals.cpu().numpy(), partials, path


@pytest.mark.parametrize("K,D,fused", [(2, 6, True), (254, 1, True), (256, 6, True), (258, 3, True),
                                       (70000, 6, True), (1 << 20, 6, True), (2500000, 6, True), (70001, 6, False),
                                       (4096, 9, False)])
def test_totals_from_the_producing_kernel(bench_devices, device_file, K, D, fused):
    """wave_scale with `partials`: the table kernel adds up each block's results itself (even K,
    D <= 8) and any other launch falls back to the first stage of the plane sum; either way the
    totals are the float64 sums of the predicted times, NaN pairs skipped, and every other output
    is what the plain call gives.  (2,500,000 kernels leave 9,766 sums per destination: the final
    stage then spreads a destination over a cluster of blocks.)"""
    kernels = workloads.make_kernels(K, seed=K + D)
    dests = (bench_devices * 2)[:D]
    out, totals, partials, path = _wave_with_partials(kernels, bench_devices[0], dests)
    assert path == "wave_scale_lut_kernel"
    assert partials.per_plane == ((K + 255) // 256 if fused else 256)
    plain = batched.wave_scale(batched.KernelBatch.from_numpy(kernels), bench_devices[0], dests)
    for name in ("scaled_ns", "dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves"):
        a, b = getattr(out, name), getattr(plain, name)
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), name
    ref = np.nansum(out.scaled_ns.cpu().numpy().astype(np.float64), axis=1)
    np.testing.assert_allclose(totals, ref, rtol=1e-13)
    np.testing.assert_allclose(totals, batched.plane_sum(out.scaled_ns).cpu().numpy(), rtol=1e-13)
    # against the oracle's float64 times: the tolerance of the float32 results
    oref = run_wave_oracle(kernels, bench_devices[0], dests)
    want = np.nansum(np.where(oref["status"] < 2, oref["scaled_ns"], np.nan), axis=1)
    np.testing.assert_allclose(totals, want, rtol=1e-6)


def test_totals_partials_edges(bench_devices):
    # the same bits from call to call, and from a partials object sized for a larger batch
    kernels = workloads.make_kernels(50000, seed=77)
    _, t1, p1, _ = _wave_with_partials(kernels, bench_devices[1], bench_devices)
    _, t2, _, _ = _wave_with_partials(kernels, bench_devices[1], bench_devices, partials=batched.WavePartials(1 << 20, 8))
    _, t3, _, _ = _wave_with_partials(kernels, bench_devices[1], bench_devices, partials=p1)
    assert np.array_equal(t1, t2) and np.array_equal(t1, t3)
    # shards cut on multiples of 256 kernels hold the same blocks: their first-stage sums are the
    # whole batch's, so the sharded total differs only by the order of the float64 additions
    parts = []
    for lo, hi in ((0, 256 * 90), (256 * 90, 50000)):
        sub = {k: v[lo:hi] for k, v in kernels.items()}
        parts.append(_wave_with_partials(sub, bench_devices[1], bench_devices)[1])
    np.testing.assert_allclose(parts[0] + parts[1], t1, rtol=1e-14)
    # per-destination register counts take the extended kernel: totals through the fallback
    g = workloads.rng(8)
    dr = torch.from_numpy(g.integers(-1, 256, size=(6, 50000)).astype(np.int16)).cuda()
    out, t4, p4, _ = _wave_with_partials(kernels, bench_devices[1], bench_devices, dest_regs=dr)
    assert p4.per_plane == 256
    np.testing.assert_allclose(t4, np.nansum(out.scaled_ns.cpu().numpy().astype(np.float64), axis=1), rtol=1e-13)
    # nothing to do: zero totals
    _, t0, p0, _ = _wave_with_partials(workloads.make_kernels(0, seed=1), bench_devices[0], bench_devices,
                                       partials=batched.WavePartials(16, 6))
    assert p0.per_plane == 0 and np.array_equal(t0, np.zeros(6))
    with pytest.raises(ValueError):
        _wave_with_partials(kernels, bench_devices[1], bench_devices, partials=batched.WavePartials(100, 6))


def test_plane_sum_scratch_is_kept_per_gpu():
    """The partial sums live in a buffer per GPU that only ever grows and is never freed while a
    launch (or a captured graph) may hold it."""
    from habitat_b200 import _native
    lib = _native.load()
    dev = torch.cuda.current_device()
    g = workloads.rng(43)
    small = torch.from_numpy(g.uniform(0, 10, size=(3, 4096)).astype(np.float32)).cuda()
    out_small = batched.plane_sum(small)
    have = lib.hb_plane_sum_scratch_planes(dev)
    assert have >= 64
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        out_graph = torch.empty(3, dtype=torch.float64, device="cuda")
        batched.plane_sum(small, out=out_graph)          # warm-up outside the capture
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            batched.plane_sum(small, out=out_graph)
    big = torch.from_numpy(g.uniform(0, 10, size=(4 * have + 1, 512)).astype(np.float32)).cuda()
    out_big = batched.plane_sum(big)                     # needs a larger buffer
    assert lib.hb_plane_sum_scratch_planes(dev) >= 4 * have + 1
    out_graph.zero_()
    graph.replay()                                       # still refers to the first buffer
    torch.cuda.synchronize()
    assert torch.equal(out_graph, out_small)
    assert np.allclose(out_big.cpu().numpy(), big.double().sum(dim=1).cpu().numpy(), rtol=1e-12)
    assert lib.hb_plane_sum_scratch_planes(-1) == -1 and lib.hb_plane_sum_scratch_planes(63) == 0


def test_index_checked_build(bench_devices):
    """The same library built with -DHB_BOUNDS_CHECK (every table and element index of the
    wave-scaling kernels compared with its bound, violations recorded, nothing traps): results equal
    the oracle's and no index is ever out of range, on the edge records and on a plain batch."""
    import os
    import subprocess
    import sys
    from habitat_b200 import build as hb_build
    if not os.path.exists(hb_build.CHECKED_LIB_PATH):
        pytest.fail("libhabitat_b200_checked.so is not built (python -m habitat_b200.build --checked)")
    code = """
import ctypes, sys
import numpy as np
sys.path.insert(0, %r)
from habitat_b200 import _native, device_table, workloads
from tests.helpers import assert_wave_equal, run_wave_gpu, run_wave_oracle
from tests.test_wave_scale_gpu import _edge_records
devs = device_table.load_device_file()
bench = [devs[n] for n in workloads.BENCH_DEVICES]
lib = _native.load()
word = ctypes.c_uint32(7)
assert lib.hb_bounds_check_word(ctypes.byref(word), 1) == 0 and word.value == 0
g = workloads.rng(5)
for kernels in (_edge_records(bench), workloads.make_kernels(20001, seed=3)):
    K = len(kernels["num_blocks"])
    regs = g.integers(-1, 300, size=(6, K)).astype(np.int16)
    for dr in (None, regs):
        got = run_wave_gpu(kernels, bench[0], bench, dest_regs=dr)
        assert got["fast_path"] == "wave_scale_lut_kernel"
        assert_wave_equal(got, run_wave_oracle(kernels, bench[0], bench, dest_regs=dr))
    got = run_wave_gpu(kernels, bench[0], bench, metrics=workloads.make_metrics(K, seed=4))
    assert got["fast_path"] == "wave_scale_lut_kernel"
from habitat_b200 import batched
kb = batched.KernelBatch.from_numpy(workloads.make_kernels(20000, seed=3))
part = batched.WavePartials(20000, 6)
out = batched.wave_scale(kb, bench[0], bench, partials=part)       # the instance that adds up its blocks' results
assert part.per_plane == 79
want = np.nansum(out.scaled_ns.cpu().numpy().astype(np.float64), axis=1)
assert np.allclose(part.totals().cpu().numpy(), want, rtol=1e-13)
assert lib.hb_bounds_check_word(ctypes.byref(word), 0) == 0
assert word.value == 0, hex(word.value)
print("checked build ok")
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, HABITAT_B200_LIB=hb_build.CHECKED_LIB_PATH)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout + r.stderr
    # the ordinary build says that it carries no checks
    from habitat_b200 import _native
    import ctypes
    assert _native.load().hb_bounds_check_word(ctypes.byref(ctypes.c_uint32(0)), 0) == _native.HB_ERR_UNSUPPORTED


def test_second_gpu_gets_its_own_tables(bench_devices):
    """One process, two GPUs: the device table and the reduction scratch are kept per GPU, so a
    launch with the other GPU current reads that GPU's own copy (uploaded at its first use)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    kernels = workloads.make_kernels(6000, seed=91)
    ref = run_wave_oracle(kernels, bench_devices[0], bench_devices)
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            got = run_wave_gpu(kernels, bench_devices[0], bench_devices)
            assert got["fast_path"] == "wave_scale_lut_kernel"
            assert_wave_equal(got, ref)
            res = batched.wave_scale(batched.KernelBatch.from_numpy(kernels, device="cuda:%d" % dev),
                                     bench_devices[0], bench_devices)
            tot = batched.plane_sum(res.scaled_ns).cpu().numpy()
            assert np.allclose(tot, np.nansum(to_numpy(res.scaled_ns).astype(np.float64), axis=1), rtol=1e-12)
