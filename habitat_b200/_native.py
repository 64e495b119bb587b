"""ctypes binding of libhabitat_b200.so (the C ABI declared in include/habitat_b200.h).

There is no fallback: if the shared library has not been built, importing this
module raises, and so does every API that needs it.
"""
import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# HABITAT_B200_LIB selects another build of the same library (the index-checked one, for tests)
LIB_PATH = os.environ.get("HABITAT_B200_LIB") or os.path.join(_PKG_DIR, "_lib", "libhabitat_b200.so")

HB_OK = 0
HB_ERR_INVALID_ARGUMENT = 1
HB_ERR_CUDA = 2
HB_ERR_UNSUPPORTED = 3
HB_ERR_DEVICE_TIMEOUT = 4
HB_ERR_TOO_LARGE = 5
HB_MAX_DEVICES = 64

HB_PAIR_LARGE, HB_PAIR_SMALL, HB_PAIR_ZERO_WAVE, HB_PAIR_BAD_INPUT = 0, 1, 2, 3
HB_PRECISION_BF16, HB_PRECISION_BF16X3 = 0, 1

DEVICE_SPEC_FIELDS = (
    "compute_major", "compute_minor", "max_threads_per_block",
    "max_threads_per_multiprocessor", "regs_per_block", "regs_per_multiprocessor",
    "warp_size", "shared_mem_per_block", "shared_mem_per_multiprocessor", "num_sms",
    "shared_mem_per_block_optin", "reserved_shared_mem_per_block", "mem_bandwidth_gb",
    "base_clock_mhz", "peak_gflops_per_second",
)


class DeviceSpec(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int32) for name in DEVICE_SPEC_FIELDS]


class KernelSoA(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "num_blocks", "block_size", "regs_per_thread", "smem_bytes", "run_time_ns", "gamma")]


class KernelMetrics(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "flop_efficiency_pct", "dram_read_bytes", "dram_write_bytes", "has_metrics")]


class WaveOut(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "scaled_ns", "dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves",
        "status", "limits")]


class HabitatNativeError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("habitat_b200 native call failed (status %d): %s" % (status, message))
        self.status = status


EXPORTS = {
    # name: (restype, argtypes)
    "hb_last_error": (ctypes.c_char_p, []),
    "hb_version": (ctypes.c_char_p, []),
    "hb_set_devices": (ctypes.c_int32, [ctypes.POINTER(DeviceSpec), ctypes.c_int32]),
    "hb_wave_scale": (ctypes.c_int32, [
        ctypes.POINTER(KernelSoA), ctypes.c_int64, ctypes.c_int32,
        ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, ctypes.c_void_p,
        ctypes.POINTER(WaveOut), ctypes.c_void_p]),
    "hb_wave_scale_metrics": (ctypes.c_int32, [
        ctypes.POINTER(KernelSoA), ctypes.POINTER(KernelMetrics), ctypes.c_int64, ctypes.c_int32,
        ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, ctypes.c_void_p,
        ctypes.POINTER(WaveOut), ctypes.c_void_p]),
    "hb_device_info": (ctypes.c_int32, [ctypes.c_int32, ctypes.POINTER(DeviceSpec)]),
    "hb_peak_flops_test": (ctypes.c_int32, [ctypes.c_int32, ctypes.POINTER(ctypes.c_double), ctypes.c_void_p]),
    "hb_wave_scale_path": (ctypes.c_int32, []),
    "hb_wave_scale_host": (ctypes.c_int32, [
        ctypes.POINTER(KernelSoA), ctypes.c_int64, ctypes.c_int32,
        ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, ctypes.c_void_p,
        ctypes.POINTER(WaveOut)]),
    "hb_thread_block_occupancy": (ctypes.c_int32, [
        ctypes.c_int32, ctypes.c_int32, ctypes.c_uint32, ctypes.c_int32,
        ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]),
    "hb_mlp_create": (ctypes.c_int32, [
        ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
        ctypes.c_int32]),
    "hb_mlp_destroy": (None, [ctypes.c_void_p]),
    "hb_mlp_predict": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
        ctypes.c_void_p]),
    "hb_mlp_status": (ctypes.c_int32, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]),
    "hb_mlp_phase_cycles": (ctypes.c_int32, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)]),
    "hb_mlp_predict_host": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]),
    "hb_special_scale": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
        ctypes.c_void_p, ctypes.c_void_p]),
    "hb_segment_sum": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
    "hb_plane_sum": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "hb_plane_sum_static": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "hb_plane_sum_scratch_planes": (ctypes.c_int64, [ctypes.c_int32]),
    "hb_group_sum": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "hb_mlp_inject_status": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_int32]),
    "hb_bounds_check_word": (ctypes.c_int32, [ctypes.POINTER(ctypes.c_uint32), ctypes.c_int32]),
    "hb_peer_create": (ctypes.c_int32, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int32]),
    "hb_peer_export": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_void_p]),
    "hb_peer_connect": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_void_p]),
    "hb_peer_connect_pointers": (ctypes.c_int32, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]),
    "hb_peer_mailbox": (ctypes.c_void_p, [ctypes.c_void_p]),
    "hb_peer_set_wait_ns": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_int64]),
    "hb_peer_destroy": (None, [ctypes.c_void_p]),
    "hb_peer_status": (ctypes.c_int32, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]),
    "hb_plane_sum_allreduce": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "hb_group_sum_allreduce": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p,
        ctypes.c_void_p]),
    "hb_wave_scale_partials_len": (ctypes.c_int64, [ctypes.c_int64]),
    "hb_wave_scale_partials": (ctypes.c_int32, [
        ctypes.POINTER(KernelSoA), ctypes.c_int64, ctypes.c_int32,
        ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, ctypes.c_void_p,
        ctypes.POINTER(WaveOut), ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.c_void_p]),
    "hb_partials_sum": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "hb_partials_sum_allreduce": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "hb_peer_allreduce": (ctypes.c_int32, [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]),
}

_lib = None


def load():
    """Loads the shared library (once) and declares every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "habitat_b200: %s is missing. Build it with `python -m habitat_b200.build` "
            "(needs nvcc); there is no CPU fallback." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in EXPORTS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status):
    if status != HB_OK:
        raise HabitatNativeError(status, load().hb_last_error().decode("utf-8", "replace"))


def current_stream_ptr():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
