"""The C ABI as a contract: every function include/habitat_b200.h declares is exported by
the built library and bound in habitat_b200/_native.py (no compute calls: CPU only)."""
import ctypes
import os
import re

import pytest

from habitat_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "habitat_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("hb_set_devices", "hb_wave_scale", "hb_wave_scale_metrics", "hb_wave_scale_host",
                 "hb_thread_block_occupancy", "hb_mlp_create", "hb_mlp_destroy", "hb_mlp_predict",
                 "hb_mlp_predict_host", "hb_mlp_status", "hb_special_scale", "hb_segment_sum",
                 "hb_plane_sum", "hb_last_error", "hb_version"):
        assert must in names


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_native.LIB_PATH):
        pytest.fail("libhabitat_b200.so is not built (python -m habitat_b200.build)")
    lib = ctypes.CDLL(_native.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), "library does not export %s" % name


def test_binding_covers_every_declared_symbol():
    declared = set(declared_functions())
    bound = set(_native.EXPORTS)
    assert declared == bound, (declared - bound, bound - declared)
    lib = _native.load()
    assert lib.hb_version().decode().count(".") == 2
    assert lib.hb_last_error() is not None


def test_struct_layouts_match_the_header():
    assert ctypes.sizeof(_native.DeviceSpec) == 15 * 4
    assert ctypes.sizeof(_native.KernelSoA) == 6 * ctypes.sizeof(ctypes.c_void_p)
    assert ctypes.sizeof(_native.KernelMetrics) == 4 * ctypes.sizeof(ctypes.c_void_p)
    assert ctypes.sizeof(_native.WaveOut) == 7 * ctypes.sizeof(ctypes.c_void_p)
    text = open(HEADER).read()
    fields = re.search(r"typedef struct \{(.*?)\} hb_device_spec;", text, flags=re.S).group(1)
    names = re.findall(r"int32_t\s+(\w+);", fields)
    assert tuple(names) == _native.DEVICE_SPEC_FIELDS


def test_partials_buffer_size_and_argument_checks():
    """Host-only parts of the totals entry points: the buffer size per destination (one sum per
    256 kernels, never fewer than the 256 sums of the fallback) and the refusal of bad arguments
    before anything touches a GPU."""
    lib = _native.load()
    sizes = {0: 256, 1: 256, 65536: 256, 65538: 257, 1 << 20: 4096, 11184812: 43691}
    for k, want in sizes.items():
        assert lib.hb_wave_scale_partials_len(k) == want
    assert lib.hb_wave_scale_partials_len(-1) == -1
    assert lib.hb_partials_sum(None, 4, 2, None, None) == _native.HB_ERR_INVALID_ARGUMENT
    assert lib.hb_partials_sum(None, -1, 0, None, None) == _native.HB_ERR_INVALID_ARGUMENT
    assert lib.hb_partials_sum(None, 0, 0, None, None) == 0          # nothing to do
    assert b"hb_partials_sum" in lib.hb_last_error()
