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
