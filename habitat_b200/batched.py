"""Batched device entry points over torch CUDA tensors.

Thin wrappers that hand raw device pointers and the current CUDA stream to the
C ABI (include/habitat_b200.h).  torch is used for device memory and streams
only; all arithmetic happens in the library's sm_100a kernels.
"""
import ctypes
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from habitat_b200 import _native, device_table


def _require_cuda(t, dtype, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError("%s must be a CUDA tensor" % name)
    if t.dtype != dtype:
        raise TypeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    return t


# HABITAT_B200_NVTX=1 wraps every native call in an NVTX range named after it, so that a timeline
# shows which entry point a kernel belongs to.
_NVTX = os.environ.get("HABITAT_B200_NVTX", "") not in ("", "0")


class _Range:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if _NVTX:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if _NVTX:
            torch.cuda.nvtx.range_pop()


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


@dataclass
class KernelBatch:
    """Structure-of-arrays view of K recorded kernels (device tensors).

    num_blocks int32, block_size uint16, regs_per_thread uint16, smem_bytes
    uint32 (static + dynamic), run_time_ns float32, gamma float32 in [0, 1].
    """
    num_blocks: torch.Tensor
    block_size: torch.Tensor
    regs_per_thread: torch.Tensor
    smem_bytes: torch.Tensor
    run_time_ns: torch.Tensor
    gamma: Optional[torch.Tensor] = None

    def __len__(self):
        return int(self.num_blocks.numel())

    @classmethod
    def from_numpy(cls, arrays, device="cuda"):
        """arrays: mapping with the six field names (numpy); uploads them."""
        def up(name, dt):
            a = np.ascontiguousarray(arrays[name]).astype(dt, copy=False)
            return torch.from_numpy(a.view(_NP_VIEW.get(dt, dt))).to(device).view(_TORCH_DT[dt])
        g = arrays.get("gamma")
        return cls(up("num_blocks", np.int32), up("block_size", np.uint16),
                   up("regs_per_thread", np.uint16), up("smem_bytes", np.uint32),
                   up("run_time_ns", np.float32),
                   up("gamma", np.float32) if g is not None else None)


_NP_VIEW = {np.uint16: np.int16, np.uint32: np.int32}
_TORCH_DT = {np.int32: torch.int32, np.uint16: torch.uint16, np.uint32: torch.uint32,
             np.float32: torch.float32}


@dataclass
class KernelMetricsBatch:
    """Raw metrics per kernel (float64 device tensors; has_metrics uint8)."""
    flop_efficiency_pct: torch.Tensor
    dram_read_bytes: torch.Tensor
    dram_write_bytes: torch.Tensor
    has_metrics: torch.Tensor


@dataclass
class WaveResult:
    """Destination-major planes: element (d, k) of a [D, K] tensor."""
    scaled_ns: torch.Tensor          # [D, K] float32, NaN where the reference raises
    dest_occupancy: torch.Tensor     # [D, K] uint8
    dest_waves: torch.Tensor         # [D, K] uint32
    origin_occupancy: torch.Tensor   # [K] uint8
    origin_waves: torch.Tensor       # [K] uint32
    status: Optional[torch.Tensor] = None   # [D, K] uint8
    limits: Optional[torch.Tensor] = None   # [D + 1, 4, K] int32


class WavePartials:
    """Room for the first stage of the per-destination totals of a wave_scale call over up to K
    kernels and D destinations (hb_wave_scale_partials): pass it as `partials=`, then `totals()`
    (or PeerTotals.partials_sum across GPUs) gives the D float64 totals without a second pass over
    the [D, K] results when the launch takes the table kernel."""

    def __init__(self, K, D, device="cuda"):
        self.K, self.D = int(K), int(D)
        n = int(_native.load().hb_wave_scale_partials_len(self.K))
        self.buffer = torch.empty((self.D * n,), dtype=torch.float64, device=device)
        self.per_plane = 0      # first-stage sums per destination left by the last call
        self.n_planes = 0

    def totals(self, out=None):
        """[D] float64 totals of the last wave_scale call that was given this object."""
        if out is None:
            out = torch.empty((self.n_planes,), dtype=torch.float64, device=self.buffer.device)
        _require_cuda(out, torch.float64, "out")
        if out.numel() != self.n_planes:
            raise ValueError("out must have one entry per destination")
        with _Range("hb_partials_sum"):
            _native.check(_native.load().hb_partials_sum(_ptr(self.buffer), self.per_plane, self.n_planes,
                                                         _ptr(out), _native.current_stream_ptr()))
        return out


def wave_scale(kernels: KernelBatch, origin, dests: Sequence, dest_regs=None, metrics=None,
               want_status=False, want_limits=False, out: Optional[WaveResult] = None,
               partials: Optional[WavePartials] = None):
    """Wave-scales K kernels measured on `origin` to every device in `dests`.

    origin / dests are DeviceProperties.  dest_regs is an optional [D, K] int16
    tensor of per-destination register counts (-1: use the kernel's own).
    With `metrics`, gamma is computed on the device per (kernel, destination).
    With `partials` the call also leaves the first stage of the per-destination totals there.
    Queued on the current stream; does not synchronise.
    """
    lib = _native.load()
    K = len(kernels)
    D = len(dests)
    dev = kernels.num_blocks.device
    _require_cuda(kernels.num_blocks, torch.int32, "num_blocks")
    _require_cuda(kernels.block_size, torch.uint16, "block_size")
    _require_cuda(kernels.regs_per_thread, torch.uint16, "regs_per_thread")
    _require_cuda(kernels.smem_bytes, torch.uint32, "smem_bytes")
    _require_cuda(kernels.run_time_ns, torch.float32, "run_time_ns")
    for name in ("block_size", "regs_per_thread", "smem_bytes", "run_time_ns"):
        if getattr(kernels, name).numel() != K:
            raise ValueError("%s has a different length" % name)
    if metrics is None:
        if kernels.gamma is None:
            raise ValueError("gamma is required unless metrics are given")
        _require_cuda(kernels.gamma, torch.float32, "gamma")
    if dest_regs is not None:
        _require_cuda(dest_regs, torch.int16, "dest_regs")
        if tuple(dest_regs.shape) != (D, K):
            raise ValueError("dest_regs must be [D, K]")
    rows = device_table.rows_of([origin] + list(dests))
    if out is None:
        out = WaveResult(
            scaled_ns=torch.empty((D, K), dtype=torch.float32, device=dev),
            dest_occupancy=torch.empty((D, K), dtype=torch.uint8, device=dev),
            dest_waves=torch.empty((D, K), dtype=torch.uint32, device=dev),
            origin_occupancy=torch.empty((K,), dtype=torch.uint8, device=dev),
            origin_waves=torch.empty((K,), dtype=torch.uint32, device=dev),
            status=torch.empty((D, K), dtype=torch.uint8, device=dev) if want_status else None,
            limits=torch.empty((D + 1, 4, K), dtype=torch.int32, device=dev) if want_limits else None)
    soa = _native.KernelSoA(_ptr(kernels.num_blocks), _ptr(kernels.block_size),
                            _ptr(kernels.regs_per_thread), _ptr(kernels.smem_bytes),
                            _ptr(kernels.run_time_ns), _ptr(kernels.gamma))
    wout = _native.WaveOut(_ptr(out.scaled_ns), _ptr(out.dest_occupancy), _ptr(out.dest_waves),
                           _ptr(out.origin_occupancy), _ptr(out.origin_waves), _ptr(out.status),
                           _ptr(out.limits))
    dest_rows = (ctypes.c_int32 * D)(*rows[1:])
    stream = _native.current_stream_ptr()
    if partials is not None:
        if metrics is not None:
            raise ValueError("partials are not available together with metrics")
        if K > partials.K or D > partials.D:
            raise ValueError("partials were sized for fewer kernels or destinations")
        per_plane = ctypes.c_int32(0)
        with _Range("hb_wave_scale_partials"):
            st = lib.hb_wave_scale_partials(ctypes.byref(soa), K, rows[0], dest_rows, D, _ptr(dest_regs),
                                            ctypes.byref(wout), _ptr(partials.buffer), ctypes.byref(per_plane),
                                            stream)
        partials.per_plane, partials.n_planes = int(per_plane.value), D
    elif metrics is None:
        with _Range("hb_wave_scale"):
            st = lib.hb_wave_scale(ctypes.byref(soa), K, rows[0], dest_rows, D, _ptr(dest_regs),
                                   ctypes.byref(wout), stream)
    else:
        _require_cuda(metrics.flop_efficiency_pct, torch.float64, "flop_efficiency_pct")
        _require_cuda(metrics.dram_read_bytes, torch.float64, "dram_read_bytes")
        _require_cuda(metrics.dram_write_bytes, torch.float64, "dram_write_bytes")
        _require_cuda(metrics.has_metrics, torch.uint8, "has_metrics")
        m = _native.KernelMetrics(_ptr(metrics.flop_efficiency_pct), _ptr(metrics.dram_read_bytes),
                                  _ptr(metrics.dram_write_bytes), _ptr(metrics.has_metrics))
        with _Range("hb_wave_scale_metrics"):
            st = lib.hb_wave_scale_metrics(ctypes.byref(soa), ctypes.byref(m), K, rows[0], dest_rows, D,
                                           _ptr(dest_regs), ctypes.byref(wout), stream)
    _native.check(st)
    return out


WAVE_PATHS = {0: "none", 1: "wave_scale_kernel", 2: "wave_scale_fast_kernel", 4: "wave_scale_lut_kernel"}


def wave_scale_path():
    """Name of the kernel the calling thread's last wave_scale call launched."""
    return WAVE_PATHS[int(_native.load().hb_wave_scale_path())]


def wave_scale_host(arrays, origin, dests, want_status=False, want_limits=False):
    """Host-buffer path: numpy in, numpy out, transfers inside the native call."""
    lib = _native.load()
    nb = np.ascontiguousarray(arrays["num_blocks"], dtype=np.int32)
    bs = np.ascontiguousarray(arrays["block_size"], dtype=np.uint16)
    rg = np.ascontiguousarray(arrays["regs_per_thread"], dtype=np.uint16)
    sm = np.ascontiguousarray(arrays["smem_bytes"], dtype=np.uint32)
    tm = np.ascontiguousarray(arrays["run_time_ns"], dtype=np.float32)
    gm = np.ascontiguousarray(arrays["gamma"], dtype=np.float32)
    K, D = nb.shape[0], len(dests)
    rows = device_table.rows_of([origin] + list(dests))
    res = dict(
        scaled_ns=np.empty((D, K), np.float32), dest_occupancy=np.empty((D, K), np.uint8),
        dest_waves=np.empty((D, K), np.uint32), origin_occupancy=np.empty((K,), np.uint8),
        origin_waves=np.empty((K,), np.uint32),
        status=np.empty((D, K), np.uint8) if want_status else None,
        limits=np.empty((D + 1, 4, K), np.int32) if want_limits else None)
    p = lambda a: ctypes.c_void_p(a.ctypes.data) if a is not None else ctypes.c_void_p(0)
    soa = _native.KernelSoA(p(nb), p(bs), p(rg), p(sm), p(tm), p(gm))
    wout = _native.WaveOut(p(res["scaled_ns"]), p(res["dest_occupancy"]), p(res["dest_waves"]),
                           p(res["origin_occupancy"]), p(res["origin_waves"]), p(res["status"]),
                           p(res["limits"]))
    dest_rows = (ctypes.c_int32 * D)(*rows[1:])
    _native.check(lib.hb_wave_scale_host(ctypes.byref(soa), K, rows[0], dest_rows, D,
                                         ctypes.c_void_p(0), ctypes.byref(wout)))
    return res


class MLPHandle:
    """Device-side weight pack of one runtime predictor (hb_mlp)."""

    def __init__(self, n_op_features, fc1_w, fc1_b, hidden_w, hidden_b, fc2_w, fc2_b, mu, sigma,
                 device_features, precision="bf16"):
        lib = _native.load()
        f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
        f64 = lambda a: np.ascontiguousarray(a, dtype=np.float64)
        fc1_w, fc1_b, hidden_w, hidden_b = f32(fc1_w), f32(fc1_b), f32(hidden_w), f32(hidden_b)
        fc2_w, fc2_b = f32(fc2_w).reshape(-1), f32(fc2_b).reshape(-1)
        mu, sigma, device_features = f64(mu), f64(sigma), f64(device_features)
        layers, width = hidden_w.shape[0], hidden_w.shape[1]
        if fc1_w.shape != (width, n_op_features + 4):
            raise ValueError("fc1 weight must be [width, F + 4]")
        if mu.shape != (n_op_features + 4,) or sigma.shape != (n_op_features + 4,):
            raise ValueError("mu and sigma must have F + 4 entries")
        if device_features.ndim != 2 or device_features.shape[1] != 4:
            raise ValueError("device_features must be [n, 4]")
        prec = {"bf16": _native.HB_PRECISION_BF16, "bf16x3": _native.HB_PRECISION_BF16X3}[precision]
        self.n_op_features = n_op_features
        self.precision = precision
        self.n_device_rows = device_features.shape[0]
        self._handle = ctypes.c_void_p(0)
        p = lambda a: ctypes.c_void_p(a.ctypes.data)
        _native.check(lib.hb_mlp_create(
            ctypes.byref(self._handle), n_op_features, layers, width, p(fc1_w), p(fc1_b),
            p(hidden_w), p(hidden_b), p(fc2_w), p(fc2_b), p(mu), p(sigma), p(device_features),
            device_features.shape[0], prec))

    def predict(self, op_features, device_row, out=None):
        """op_features [Q, F] float32 CUDA, device_row [Q] uint8 CUDA -> [Q] float32."""
        lib = _native.load()
        _require_cuda(op_features, torch.float32, "op_features")
        _require_cuda(device_row, torch.uint8, "device_row")
        Q = op_features.shape[0]
        if op_features.ndim != 2 or op_features.shape[1] != self.n_op_features:
            raise ValueError("op_features must be [Q, %d]" % self.n_op_features)
        if device_row.numel() != Q:
            raise ValueError("device_row must have Q entries")
        if out is None:
            out = torch.empty((Q,), dtype=torch.float32, device=op_features.device)
        with _Range("hb_mlp_predict"):
            _native.check(lib.hb_mlp_predict(self._handle, _ptr(op_features), _ptr(device_row), Q,
                                             _ptr(out), _native.current_stream_ptr()))
        return out

    def predict_host(self, op_features, device_row):
        """numpy in / numpy out; transfers and the status check inside the native call."""
        lib = _native.load()
        f = np.ascontiguousarray(op_features, dtype=np.float32)
        r = np.ascontiguousarray(device_row, dtype=np.uint8)
        out = np.empty((f.shape[0],), np.float32)
        _native.check(lib.hb_mlp_predict_host(
            self._handle, ctypes.c_void_p(f.ctypes.data), ctypes.c_void_p(r.ctypes.data),
            f.shape[0], ctypes.c_void_p(out.ctypes.data)))
        return out

    def check_status(self):
        """Synchronises and raises if a launch gave up on a bounded device wait (reported once:
        the next call judges the launches after this one)."""
        code = ctypes.c_int32(0)
        _native.check(_native.load().hb_mlp_status(self._handle, ctypes.byref(code)))

    def inject_status(self, code):
        """Writes the device status word from the host (tests of the error path)."""
        _native.check(_native.load().hb_mlp_inject_status(self._handle, int(code)))

    def phase_cycles(self):
        """Cycle counters of the first cluster in the last bf16 launch (synchronises): epilogue group 0
        (wait, epilogue, fc2, layers, epi_publish, epi_remote), the MMA issuer (mma_wait_act,
        mma_wait_weights, mma_wait_tmem, mma_issue, slots; mma_total_cycles and mma_total_ns over the
        same interval, whose ratio is the SM clock under load) and the first producer."""
        out = (ctypes.c_int64 * 16)()
        _native.check(_native.load().hb_mlp_phase_cycles(self._handle, out))
        names = ("wait", "epilogue", "fc2", "layers", "mma_wait_act", "mma_wait_weights", "mma_wait_tmem",
                 "mma_issue", "slots", "producer_wait_slot", "producer_copy", "copies", "mma_total_cycles",
                 "mma_total_ns", "epi_publish", "epi_remote")
        return dict(zip(names, [int(x) for x in out]))

    def close(self):
        if self._handle:
            _native.load().hb_mlp_destroy(self._handle)
            self._handle = ctypes.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def special_scale(run_time_ms, pred_dest, pred_orig, negative_count=None):
    """max(0, run_time_ms * pred_dest / pred_orig) elementwise (float32 CUDA tensors)."""
    lib = _native.load()
    for name, t in (("run_time_ms", run_time_ms), ("pred_dest", pred_dest), ("pred_orig", pred_orig)):
        _require_cuda(t, torch.float32, name)
    n = run_time_ms.numel()
    out = torch.empty_like(run_time_ms)
    if negative_count is not None:
        _require_cuda(negative_count, torch.uint32, "negative_count")
    _native.check(lib.hb_special_scale(_ptr(run_time_ms), _ptr(pred_dest), _ptr(pred_orig), n,
                                       _ptr(out), _ptr(negative_count), _native.current_stream_ptr()))
    return out


def segment_sum(values, offsets):
    """float64 sums of values[offsets[s]:offsets[s+1]] (float32 / int64 CUDA tensors)."""
    lib = _native.load()
    _require_cuda(values, torch.float32, "values")
    _require_cuda(offsets, torch.int64, "offsets")
    n = offsets.numel() - 1
    out = torch.empty((max(n, 0),), dtype=torch.float64, device=values.device)
    _native.check(lib.hb_segment_sum(_ptr(values), _ptr(offsets), n, _ptr(out),
                                     _native.current_stream_ptr()))
    return out


def plane_sum(values, out=None):
    """float64 sum of each row of a [P, L] float32 CUDA tensor, NaN entries skipped."""
    lib = _native.load()
    _require_cuda(values, torch.float32, "values")
    if values.ndim != 2:
        raise ValueError("values must be [planes, length]")
    P, L = values.shape
    if out is None:
        out = torch.empty((P,), dtype=torch.float64, device=values.device)
    else:
        _require_cuda(out, torch.float64, "out")
        if out.numel() != P:
            raise ValueError("out must have one entry per plane")
    _native.check(lib.hb_plane_sum(_ptr(values), L, P, _ptr(out), _native.current_stream_ptr()))
    return out


def group_sum(values, keys, n_groups, out=None):
    """float64 sums of a float32 CUDA vector grouped by a uint8 key per element (keys at or above
    n_groups and NaN values are skipped): per-device totals of a batch of MLP predictions."""
    lib = _native.load()
    _require_cuda(values, torch.float32, "values")
    _require_cuda(keys, torch.uint8, "keys")
    if values.numel() != keys.numel():
        raise ValueError("values and keys must have the same length")
    if out is None:
        out = torch.empty((n_groups,), dtype=torch.float64, device=values.device)
    else:
        _require_cuda(out, torch.float64, "out")
        if out.numel() != n_groups:
            raise ValueError("out must have one entry per group")
    _native.check(lib.hb_group_sum(_ptr(values), _ptr(keys), values.numel(), n_groups, _ptr(out),
                                   _native.current_stream_ptr()))
    return out
