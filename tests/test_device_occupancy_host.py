"""The library's occupancy code, compiled for the host, against the oracle (CPU only)."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from habitat_b200 import _native
from oracle import wave as owave

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("harness") / "libocc_harness.so")
    subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared",
                    "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "habitat_b200", "csrc"),
                    os.path.join(HERE, "occupancy_host_harness.cpp"), "-o", out], check=True)
    lib = ctypes.CDLL(out)
    lib.harness_occupancy.restype = None
    lib.harness_fast_occupancy.restype = None
    lib.harness_magic_errors.restype = ctypes.c_long
    lib.harness_lut.restype = ctypes.c_int
    lib.harness_tables.restype = ctypes.c_int
    return lib


def _run(harness, spec, block, smem, regs):
    n = len(block)
    d = _native.DeviceSpec(*[int(v) for v in spec])
    occ = np.empty(n, np.int32)
    lim = np.empty((n, 4), np.int32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    harness.harness_occupancy(ctypes.byref(d), ctypes.c_long(n), p(block), p(smem), p(regs), p(occ), p(lim))
    fast = np.empty(n, np.int32)
    harness.harness_fast_occupancy(ctypes.byref(d), ctypes.c_long(n), p(block), p(smem), p(regs), p(fast))
    if (fast >= 0).any():
        # the division-free form must agree wherever the row qualifies for it
        assert np.array_equal(fast, occ), "fast path disagrees"
    return occ, lim


@pytest.mark.parametrize("seed", [0, 1])
def test_all_rows_random(harness, device_file, seed):
    g = np.random.Generator(np.random.PCG64(100 + seed))
    n = 20000
    block = g.integers(1, 1100, n).astype(np.int32)
    regs = g.integers(0, 300, n).astype(np.int32)
    smem = g.integers(0, 240 * 1024, n).astype(np.int32)
    for name, dev in device_file.items():
        spec = dev.spec_tuple()
        occ, lim = _run(harness, spec, block, smem, regs)
        for i in range(n):
            o, l = owave.occupancy(spec, block[i], smem[i], regs[i])
            assert occ[i] == o and list(lim[i]) == l, (name, block[i], smem[i], regs[i])


def test_odd_device_rows(harness):
    """Rows the tables never contain: unknown architectures, non-positive
    fields, a warp size that is not a power of two, a carve-out below the cap."""
    base = dict(zip(_native.DEVICE_SPEC_FIELDS,
                    (7, 0, 1024, 2048, 65536, 65536, 32, 49152, 98304, 80, 0, 0, 900, 1530, 15700)))
    variants = [dict(compute_major=4), dict(compute_major=11), dict(compute_major=10, compute_minor=2),
                dict(compute_major=12, compute_minor=3), dict(warp_size=0), dict(num_sms=0),
                dict(warp_size=48), dict(shared_mem_per_multiprocessor=16384),
                dict(compute_major=8, compute_minor=0, shared_mem_per_multiprocessor=200 * 1024,
                     reserved_shared_mem_per_block=1024),
                dict(compute_major=8, compute_minor=9, reserved_shared_mem_per_block=1024,
                     shared_mem_per_multiprocessor=100 * 1024, shared_mem_per_block=120 * 1024),
                dict(compute_major=3, compute_minor=5), dict(compute_major=5, compute_minor=2),
                dict(regs_per_block=32768), dict(compute_major=6, compute_minor=0, regs_per_block=32768)]
    g = np.random.Generator(np.random.PCG64(5))
    n = 4000
    block = g.integers(1, 1100, n).astype(np.int32)
    regs = g.integers(0, 300, n).astype(np.int32)
    smem = g.integers(0, 130 * 1024, n).astype(np.int32)
    for v in variants:
        spec = tuple({**base, **v}[f] for f in _native.DEVICE_SPEC_FIELDS)
        occ, lim = _run(harness, spec, block, smem, regs)
        for i in range(n):
            o, l = owave.occupancy(spec, block[i], smem[i], regs[i])
            assert occ[i] == o and list(lim[i]) == l, (v, block[i], smem[i], regs[i])


def test_magic_division(harness):
    assert harness.harness_magic_errors() == 0


def test_fast_path_covers_shipped_rows(harness, device_file):
    g = np.random.Generator(np.random.PCG64(8))
    block = g.integers(1, 1100, 100).astype(np.int32)
    regs = g.integers(0, 300, 100).astype(np.int32)
    smem = g.integers(0, 100000, 100).astype(np.int32)
    for name, dev in device_file.items():
        d = _native.DeviceSpec(*[int(v) for v in dev.spec_tuple()])
        fast = np.empty(100, np.int32)
        p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        harness.harness_fast_occupancy(ctypes.byref(d), ctypes.c_long(100), p(block), p(smem), p(regs), p(fast))
        assert (fast >= 0).all(), name


def _run_lut(harness, spec, block, smem, regs, nb):
    """Occupancy and wave counts as the table kernel forms them, from the tables built for `spec`."""
    n = len(block)
    d = _native.DeviceSpec(*[int(v) for v in spec])
    occ, waves = np.empty(n, np.int32), np.empty(n, np.uint32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    ok = harness.harness_lut(ctypes.byref(d), ctypes.c_long(n), p(block), p(smem), p(regs), p(nb), p(occ), p(waves))
    return bool(ok), occ, waves


def test_tables_of_every_shipped_row(harness, device_file):
    """The P / S / T tables the library builds per device row, read the way the table kernel reads
    them, against the oracle: every warps-per-block and register step, every 128-byte step of shared
    memory around its edges, and the exact multiply-shift division on grid sizes up to 2^31 - 1."""
    g = np.random.Generator(np.random.PCG64(31))
    block = np.concatenate([np.arange(0, 1100), g.integers(0, 1100, 6000), [2048, 65535]]).astype(np.int32)
    n = len(block)
    regs = np.concatenate([np.arange(0, 330), g.integers(0, 300, n - 330)]).astype(np.int32)
    smem = np.concatenate([np.arange(0, 2050) * 128, np.arange(1, 2051) * 128 - 1, np.arange(0, 2050) * 128 + 1,
                           g.integers(0, 240 * 1024, n - 3 * 2050)])[:n].astype(np.uint32)
    smem[-4:] = [0xFFFFFFFF, 0x80000000, 0x7FFF0001, 0x7FFF0000]
    nb = np.concatenate([g.integers(1, 2 ** 31 - 1, n - 6), [1, 2, 2 ** 31 - 1, 2 ** 31 - 2, 2 ** 30, 12345]]).astype(np.int32)
    tabulated = 0
    for name, dev in device_file.items():
        spec = dev.spec_tuple()
        ok, occ, waves = _run_lut(harness, spec, block, smem, regs, nb)
        if not ok:
            continue
        tabulated += 1
        for i in range(n):
            sm = -1 if smem[i] > 0x7FFF0000 else int(smem[i])
            o, _ = owave.occupancy(spec, block[i], sm, regs[i])
            assert occ[i] == o, (name, block[i], smem[i], regs[i])
            if o:
                assert waves[i] == int(nb[i]) // (dev.num_sms * o), (name, nb[i], o)
    assert tabulated >= 8


def test_tables_of_fuzzed_rows(harness):
    """Property test: device rows nobody ships (odd SM counts, thread limits, carve-outs, reserves)."""
    from hypothesis import given, settings
    from hypothesis import strategies as st
    g = np.random.Generator(np.random.PCG64(32))
    n = 600
    block = g.integers(0, 1200, n).astype(np.int32)
    regs = g.integers(0, 300, n).astype(np.int32)
    smem = g.integers(0, 240 * 1024, n).astype(np.uint32)
    nb = g.integers(1, 2 ** 31 - 1, n).astype(np.int32)
    seen = {"tabulated": 0}

    @settings(max_examples=60, deadline=None)
    @given(major=st.sampled_from([3, 5, 6, 7, 8, 9, 10, 12]), minor=st.sampled_from([0, 1, 2, 5, 6, 7, 9]),
           tpb=st.sampled_from([512, 768, 1024]), tpm=st.sampled_from([1024, 1536, 2048]),
           rpb=st.sampled_from([32768, 65536]), rpm=st.sampled_from([65536, 131072]),
           spb=st.sampled_from([48 * 1024, 99 * 1024, 163 * 1024, 227 * 1024]),
           spm=st.sampled_from([64 * 1024, 96 * 1024, 100 * 1024, 164 * 1024, 228 * 1024]),
           sms=st.integers(2, 400), reserve=st.sampled_from([0, 1024]), clock=st.integers(100, 3000))
    def check(major, minor, tpb, tpm, rpb, rpm, spb, spm, sms, reserve, clock):
        spec = (major, minor, tpb, tpm, rpb, rpm, 32, spb, spm, sms, 0, reserve if major >= 8 else 0, 900, clock, 15000)
        ok, occ, waves = _run_lut(harness, spec, block, smem, regs, nb)
        if not ok:
            return
        seen["tabulated"] += 1
        for i in range(0, n, 3):
            o, _ = owave.occupancy(spec, block[i], int(smem[i]), regs[i])
            assert occ[i] == o, (spec, block[i], smem[i], regs[i])
            if o:
                assert waves[i] == int(nb[i]) // (sms * o)
    check()
    assert seen["tabulated"] >= 10


def test_host_code_under_sanitizers(tmp_path):
    """The library's host-compilable integer code and its table builder, built with
    -fsanitize=address,undefined and driven with fuzzed rows and records (the harness's main):
    an out-of-range table index or undefined arithmetic aborts the run."""
    exe = str(tmp_path / "harness_sanitized")
    subprocess.run(["g++", "-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
                    "-DHARNESS_MAIN", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "habitat_b200", "csrc"),
                    os.path.join(HERE, "occupancy_host_harness.cpp"), "-o", exe], check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "mismatched 0" in r.stdout, r.stdout + r.stderr


def test_table_kernel_arithmetic_in_float32(harness, bench_devices):
    """The float32 formulation of the table kernel, replayed in numpy from the library's own
    tables, against the float64 oracle: wave counts by multiply-shift, the small-kernel exponent
    (1 - gamma) (A_dest[m_d] - A_origin[m_o]) from hi + lo table entries, the large-kernel exponent
    from split constants, one exp2 per pair.  Guards the 1e-6 error budget without a GPU (the
    device adds the error of ex2.approx, two units in the last place)."""
    from habitat_b200 import workloads
    K = 1 << 16
    k = workloads.make_kernels(K, 1002)
    specs = [d.spec_tuple() for d in bench_devices]
    ref = owave.wave_scale_batch(specs, 0, list(range(6)), k, want_limits=False)

    def tables(spec):
        d = _native.DeviceSpec(*[int(v) for v in spec])
        P, S, T = np.empty(34 * 34, np.uint8), np.empty(2048, np.uint8), np.empty(33 * 4, np.uint32)
        p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        assert harness.harness_tables(ctypes.byref(d), p(P), p(S), p(T))
        T = T.reshape(33, 4)
        return P, S, T[:, 0].astype(np.uint64), T[:, 1].astype(np.uint64), T[:, 2].copy().view(np.float32), \
            T[:, 3].copy().view(np.float32)

    f32 = np.float32
    bs, rg, sm = k["block_size"].astype(np.uint32), k["regs_per_thread"].astype(np.uint32), k["smem_bytes"].astype(np.uint32)
    pidx = np.minimum((bs + 31) >> 5, 33) * 34 + np.minimum((rg + 7) >> 3, 33)
    sidx = (np.minimum(sm, 2047 << 7) + 127) >> 7
    nb = k["num_blocks"].astype(np.uint64)
    t, g = k["run_time_ns"].astype(f32), k["gamma"].astype(f32)
    omg = (f32(1.0) - g).astype(f32)
    tab = [tables(s) for s in specs]
    origin = bench_devices[0]

    def occ_waves(i):
        P, S, M, sh, _, _ = tab[i]
        occ = np.minimum(P[pidx], S[sidx]).astype(np.int64)
        q = ((nb * M[occ]) >> np.uint64(32)) >> sh[occ]
        return occ, q

    occ_o, q_o = occ_waves(0)
    assert np.array_equal(occ_o, ref["origin_occupancy"])
    live = occ_o > 0
    fits_o = live & (q_o == 0)
    om = np.where(fits_o, -(-nb.astype(np.int64) // origin.num_sms), 1)
    ao_hi, ao_lo = tab[0][4][om], tab[0][5][om]
    worst = 0.0
    for d, dev in enumerate(bench_devices):
        occ, q = occ_waves(d)
        assert np.array_equal(occ, ref["dest_occupancy"][d])
        has = occ > 0
        assert np.array_equal(np.where(has, q, 0xFFFFFFFF).astype(np.uint32), ref["dest_waves"][d])
        small = fits_o & has & (q == 0)
        ok = live & ~(fits_o & ~has)
        assert np.array_equal(ok, ref["status"][d] <= 1) and np.array_equal(small, ref["status"][d] == 1)
        dm = np.where(small, -(-nb.astype(np.int64) // dev.num_sms), 1)
        e_small = (omg * ((tab[d][4][dm] - ao_hi).astype(f32) + (tab[d][5][dm] - ao_lo).astype(f32)).astype(f32)).astype(f32)
        b = np.log2(origin.base_clock_mhz / dev.base_clock_mhz) + np.log2(origin.num_sms / dev.num_sms)
        a = np.log2(origin.mem_bandwidth_gb / dev.mem_bandwidth_gb) - b
        a_hi, b_hi = f32(a), f32(b)
        a_lo, b_lo = f32(a - np.float64(a_hi)), f32(b - np.float64(b_hi))
        fma = lambda x, y, z: (x.astype(np.float64) * np.float64(y) + np.float64(z)).astype(f32)
        e = np.where(small, e_small, (fma(g, a_hi, b_hi) + fma(g, a_lo, b_lo)).astype(f32))
        out = (t * np.exp2(e.astype(np.float64)).astype(f32)).astype(f32)
        err = np.abs(out[ok].astype(np.float64) - ref["scaled_ns"][d][ok]) / ref["scaled_ns"][d][ok]
        worst = max(worst, float(err.max()))
    assert worst <= 5e-7, worst          # leaves room for the device's approximate exp2 inside 1e-6
