"""The C oracle against the compiled reference and the toolkit header (CPU only).

The reference has no tests of its own; these pin the restatement in oracle/ to
the reference's C++ (compiled from its sources into oracle/_ref) wherever that
code is defined (compute capability <= 7.5), and to the CUDA toolkit's
cuda_occupancy.h under the same call convention for newer parts.
"""
import ctypes
import os

import numpy as np
import pytest

from oracle import build as obuild
from oracle import wave as owave

REF = obuild.build_ref()


class _Dev(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in owave.FIELDS]


def _load(key, fn):
    if key not in REF or not os.path.exists(REF[key]):
        pytest.skip("%s not built (reference tree absent)" % key)
    lib = ctypes.CDLL(REF[key])
    f = getattr(lib, fn)
    f.restype = None
    return f


def _samples(n, seed, edge=False):
    g = np.random.Generator(np.random.PCG64(seed))
    if edge:
        block = g.integers(1, 1100, n)
        regs = g.integers(0, 300, n)
        smem = g.integers(0, 110 * 1024, n)
    else:
        block = g.choice([32, 64, 96, 128, 192, 256, 384, 512, 768, 1024], n)
        regs = g.integers(16, 256, n)
        smem = 256 * g.integers(0, 385, n)
    return block.astype(np.int32), regs.astype(np.int32), smem.astype(np.int32)


def _oracle_batch(spec, block, smem, regs):
    occ = np.empty(len(block), np.int32)
    lim = np.empty((len(block), 4), np.int32)
    for i in range(len(block)):
        o, l = owave.occupancy(spec, block[i], smem[i], regs[i])
        occ[i], lim[i] = o, l
    return occ, lim


def _header_batch(fn, spec, block, smem, regs, split_static=False):
    n = len(block)
    d = _Dev(*[int(v) for v in spec])
    occ = np.empty(n, np.int32)
    lim = np.empty((n, 4), np.int32)
    static = (smem // 3).astype(np.int32) if split_static else np.zeros(n, np.int32)
    dyn = (smem - static).astype(np.int32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    fn(ctypes.byref(d), ctypes.c_int64(n), p(block), p(dyn), p(static), p(regs), p(occ), p(lim))
    return occ, lim


REF_ROWS = ["P4000", "GTX1080Ti", "RTX2070", "RTX2080Ti", "P4", "T4", "V100", "P100", "V100_16"]
NEW_ROWS = ["A100_40", "H100_80", "RTX3090", "B200"]


@pytest.mark.parametrize("name", REF_ROWS)
@pytest.mark.parametrize("edge", [False, True])
def test_oracle_matches_reference_header(device_file, name, edge):
    fn = _load("ref", "ref_header_limits_batch")
    spec = device_file[name].spec_tuple()
    block, regs, smem = _samples(20000, 7 + edge, edge)
    occ_o, lim_o = _oracle_batch(spec, block, smem, regs)
    occ_r, lim_r = _header_batch(fn, spec, block, smem, regs, split_static=True)
    assert np.array_equal(occ_o, occ_r)
    ok = occ_r >= 0
    assert np.array_equal(lim_o[ok], lim_r[ok])


@pytest.mark.parametrize("name", REF_ROWS)
def test_oracle_matches_reference_kernel_cpp(device_file, name):
    fn = _load("ref", "ref_thread_block_occupancy_batch")
    spec = device_file[name].spec_tuple()
    block, regs, smem = _samples(20000, 11, True)
    occ_o, _ = _oracle_batch(spec, block, smem, regs)
    d = _Dev(*[int(v) for v in spec])
    out = np.empty(len(block), np.uint32)
    zero = np.zeros(len(block), np.int32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    fn(ctypes.byref(d), ctypes.c_int64(len(block)), p(block), p(smem), p(zero), p(regs), p(out))
    assert np.array_equal(occ_o.astype(np.uint32), out)


@pytest.mark.parametrize("name", NEW_ROWS)
@pytest.mark.parametrize("edge", [False, True])
def test_oracle_matches_toolkit_header(device_file, name, edge):
    fn = _load("toolkit", "tk_header_limits_batch")
    spec = device_file[name].spec_tuple()
    block, regs, smem = _samples(20000, 13 + edge, edge)
    occ_o, lim_o = _oracle_batch(spec, block, smem, regs)
    occ_t, lim_t = _header_batch(fn, spec, block, smem, regs, split_static=True)
    assert np.array_equal(occ_o, occ_t)
    assert np.array_equal(lim_o, lim_t)


def test_reference_rejects_new_architectures(device_file):
    """The vendored header knows nothing past compute capability 7.x: Habitat
    maps that error to occupancy 0 (cpp/src/cuda/kernel.cpp:45-53)."""
    fn = _load("ref", "ref_header_limits_batch")
    block, regs, smem = _samples(256, 3)
    for name in NEW_ROWS:
        occ, _ = _header_batch(fn, device_file[name].spec_tuple(), block, smem, regs)
        assert not occ.any()


# Known answers read off the reference's own code for (V100, T4, P100, P4000);
# tuple = (block, dynamic smem, static smem, regs).
KAT = [
    ((256, 0, 0, 32), (8, 4, 8, 8)), ((256, 0, 0, 64), (4, 4, 4, 4)),
    ((1024, 0, 0, 64), (1, 1, 1, 1)), ((1024, 0, 0, 65), (0, 0, 0, 0)),
    ((128, 16384, 0, 40), (6, 4, 4, 6)), ((64, 0, 49152, 16), (2, 1, 1, 2)),
    ((64, 256, 49152, 16), (0, 0, 0, 0)), ((32, 0, 0, 16), (32, 16, 32, 32)),
    ((256, 8448, 0, 24), (8, 4, 7, 8)), ((96, 0, 40000, 72), (2, 1, 1, 2)),
]


def test_known_answers(device_file):
    for (block, dyn, static, regs), expect in KAT:
        got = tuple(owave.occupancy(device_file[n].spec_tuple(), block, dyn + static, regs)[0]
                    for n in ("V100", "T4", "P100", "P4000"))
        assert got == expect, (block, dyn, static, regs)


def test_odd_rows_against_toolkit_header():
    """Device rows outside the shipped table, for the architectures the toolkit
    header covers: unknown minors, carve-outs beyond the ladder, caps above the
    per-SM size."""
    fn = _load("toolkit", "tk_header_limits_batch")
    base = dict(zip(owave.FIELDS,
                    (8, 0, 1024, 2048, 65536, 65536, 32, 49152, 167936, 108, 0, 1024, 1555, 1410, 19500)))
    variants = [dict(compute_major=10, compute_minor=2), dict(compute_major=12, compute_minor=3),
                dict(shared_mem_per_multiprocessor=200 * 1024), dict(compute_major=11),
                dict(compute_minor=9, shared_mem_per_multiprocessor=100 * 1024,
                     shared_mem_per_block=120 * 1024),
                dict(compute_major=9, shared_mem_per_multiprocessor=16384),
                dict(compute_major=12, compute_minor=1, shared_mem_per_multiprocessor=100 * 1024),
                dict(compute_major=10, compute_minor=1, shared_mem_per_multiprocessor=228 * 1024),
                dict(compute_major=8, compute_minor=7), dict(warp_size=48), dict(regs_per_block=32768)]
    block, regs, smem = _samples(6000, 21, True)
    smem = (smem * 2).astype(np.int32)
    for v in variants:
        spec = tuple({**base, **v}[f] for f in owave.FIELDS)
        occ_o, lim_o = _oracle_batch(spec, block, smem, regs)
        occ_t, lim_t = _header_batch(fn, spec, block, smem, regs)
        assert np.array_equal(occ_o, occ_t), v
        assert np.array_equal(lim_o, lim_t), v


def test_odd_rows_against_reference_header():
    fn = _load("ref", "ref_header_limits_batch")
    base = dict(zip(owave.FIELDS,
                    (7, 0, 1024, 2048, 65536, 65536, 32, 49152, 98304, 80, 0, 0, 900, 1530, 15700)))
    variants = [dict(compute_major=4), dict(compute_major=3, compute_minor=5),
                dict(compute_major=5, compute_minor=2), dict(warp_size=0), dict(num_sms=0),
                dict(warp_size=48), dict(shared_mem_per_multiprocessor=16384),
                dict(shared_mem_per_multiprocessor=100 * 1024, shared_mem_per_block=99 * 1024),
                dict(compute_minor=5, shared_mem_per_multiprocessor=65536, shared_mem_per_block=65536),
                dict(regs_per_block=32768), dict(compute_major=6, compute_minor=0, regs_per_block=32768),
                dict(compute_major=6, compute_minor=0, regs_per_multiprocessor=32768)]
    block, regs, smem = _samples(6000, 22, True)
    for v in variants:
        spec = tuple({**base, **v}[f] for f in owave.FIELDS)
        occ_o, lim_o = _oracle_batch(spec, block, smem, regs)
        occ_r, lim_r = _header_batch(fn, spec, block, smem, regs)
        assert np.array_equal(occ_o, occ_r), v
        assert np.array_equal(lim_o, lim_r), v
