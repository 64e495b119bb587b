"""ctypes front end of the C oracle (habitat_oracle.c) -- TEST INFRASTRUCTURE ONLY."""
import ctypes
import os

import numpy as np

from oracle import build as _build

FIELDS = (
    "compute_major", "compute_minor", "max_threads_per_block",
    "max_threads_per_multiprocessor", "regs_per_block", "regs_per_multiprocessor",
    "warp_size", "shared_mem_per_block", "shared_mem_per_multiprocessor", "num_sms",
    "shared_mem_per_block_optin", "reserved_shared_mem_per_block", "mem_bandwidth_gb",
    "base_clock_mhz", "peak_gflops_per_second",
)


class Device(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in FIELDS]


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_build.BUILD_DIR, "libhabitat_oracle.so")
        if not os.path.exists(path):
            path = _build.build_oracle()
        L = ctypes.CDLL(path)
        L.hbo_occupancy.restype = ctypes.c_int
        L.hbo_occupancy.argtypes = [ctypes.POINTER(Device), ctypes.c_int, ctypes.c_int64,
                                    ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        L.hbo_roofline_gamma.restype = ctypes.c_double
        L.hbo_roofline_gamma.argtypes = [ctypes.c_double] * 4 + [ctypes.POINTER(Device)] * 2
        L.hbo_wave_scale_batch.restype = ctypes.c_int
        L.hbo_wave_scale_batch.argtypes = [
            ctypes.POINTER(Device), ctypes.c_int, ctypes.POINTER(ctypes.c_int32), ctypes.c_int,
            ctypes.c_int64] + [ctypes.c_void_p] * 14
        _lib = L
    return _lib


def device_array(spec_tuples):
    arr = (Device * len(spec_tuples))()
    for i, s in enumerate(spec_tuples):
        arr[i] = Device(*[int(v) for v in s])
    return arr


def occupancy(spec, block_size, smem_total, regs):
    """Scalar call: returns (occupancy, [regs, warps, blocks, smem] limits)."""
    d = Device(*[int(v) for v in spec])
    lim = (ctypes.c_int * 4)()
    occ = lib().hbo_occupancy(ctypes.byref(d), int(block_size), int(smem_total), int(regs), lim)
    return occ, list(lim)


def roofline_gamma(eff, rd, wr, t_ns, origin_spec, dest_spec):
    o = Device(*[int(v) for v in origin_spec])
    d = Device(*[int(v) for v in dest_spec])
    return lib().hbo_roofline_gamma(float(eff), float(rd), float(wr), float(t_ns),
                                    ctypes.byref(o), ctypes.byref(d))


def wave_scale_batch(spec_tuples, origin_row, dest_rows, kernels, dest_regs=None,
                     want_limits=True):
    """kernels: dict of numpy arrays (num_blocks, block_size, regs_per_thread,
    smem_bytes, run_time_ns float64, gamma float32).  Returns a dict of numpy
    arrays shaped like the device path's outputs, plus `threads`."""
    devs = device_array(spec_tuples)
    nb = np.ascontiguousarray(kernels["num_blocks"], dtype=np.int32)
    bs = np.ascontiguousarray(kernels["block_size"], dtype=np.uint16)
    rg = np.ascontiguousarray(kernels["regs_per_thread"], dtype=np.uint16)
    sm = np.ascontiguousarray(kernels["smem_bytes"], dtype=np.uint32)
    tm = np.ascontiguousarray(kernels["run_time_ns"], dtype=np.float64)
    gm = np.ascontiguousarray(kernels["gamma"], dtype=np.float32)
    K, D = nb.shape[0], len(dest_rows)
    out = dict(
        scaled_ns=np.empty((D, K), np.float64), dest_occupancy=np.empty((D, K), np.uint8),
        dest_waves=np.empty((D, K), np.uint32), origin_occupancy=np.empty((K,), np.uint8),
        origin_waves=np.empty((K,), np.uint32), status=np.empty((D, K), np.uint8),
        limits=np.empty((D + 1, 4, K), np.int32) if want_limits else None)
    dr = None if dest_regs is None else np.ascontiguousarray(dest_regs, dtype=np.int16)
    p = lambda a: ctypes.c_void_p(a.ctypes.data) if a is not None else ctypes.c_void_p(0)
    rows = (ctypes.c_int32 * D)(*[int(r) for r in dest_rows])
    out["threads"] = lib().hbo_wave_scale_batch(
        devs, int(origin_row), rows, D, K, p(nb), p(bs), p(rg), p(sm), p(tm), p(gm), p(dr),
        p(out["scaled_ns"]), p(out["dest_occupancy"]), p(out["dest_waves"]),
        p(out["origin_occupancy"]), p(out["origin_waves"]), p(out["status"]), p(out["limits"]))
    return out


def wave_scale_pair(origin_spec, dest_spec, num_blocks, block_size, smem_total, regs, dest_regs,
                    run_time_ns, gamma):
    """One pair with a float64 gamma: returns (status, scaled_ns, origin_occ, dest_occ)."""
    L = lib()
    if not getattr(L, "_pair_ready", False):
        L.hbo_wave_scale_pair.restype = ctypes.c_int
        L.hbo_wave_scale_pair.argtypes = [
            ctypes.POINTER(Device), ctypes.POINTER(Device), ctypes.c_int32, ctypes.c_int,
            ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_double,
            ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
            ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
        L._pair_ready = True
    o = Device(*[int(v) for v in origin_spec])
    d = Device(*[int(v) for v in dest_spec])
    out = ctypes.c_double()
    oo, od = ctypes.c_int(), ctypes.c_int()
    wo, wd = ctypes.c_int64(), ctypes.c_int64()
    st = L.hbo_wave_scale_pair(ctypes.byref(o), ctypes.byref(d), int(num_blocks), int(block_size),
                               int(smem_total), int(regs), int(dest_regs), float(run_time_ns),
                               float(gamma), ctypes.byref(out), ctypes.byref(oo), ctypes.byref(od),
                               ctypes.byref(wo), ctypes.byref(wd))
    return st, out.value, oo.value, od.value
