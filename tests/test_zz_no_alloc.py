"""hb_plane_sum_static: the plane sum that never allocates.

Some hosts of this library may not allocate device memory once they are up (the
whole GPU belongs to their own pool, or their latency rules forbid driver
allocations while serving).  For them the library carries its scratch inside its
own image.  The entry point must give exactly what hb_plane_sum gives - the two
run the same kernels, only the scratch differs - on consecutive calls that reuse
the shared scratch, and must refuse more planes than the scratch holds.

Collected last on purpose: if it fails, every other test has already run.
"""
import ctypes

import numpy as np
import pytest
import torch

from habitat_b200 import _native, batched, workloads

pytestmark = pytest.mark.gpu


def _static_sum(values, out):
    lib = _native.load()
    return lib.hb_plane_sum_static(ctypes.c_void_p(values.data_ptr()), values.shape[1], values.shape[0],
                                   ctypes.c_void_p(out.data_ptr()), _native.current_stream_ptr())


def test_matches_allocating_entry_point_twice_in_a_row():
    g = workloads.rng(91)
    for planes, length in ((6, 1 << 20), (64, 4099), (1, 7)):     # second call reuses dirty scratch
        host = g.uniform(0, 5e6, size=(planes, length)).astype(np.float32)
        host[:, ::11] = np.nan                                     # pairs the reference raises on
        values = torch.from_numpy(host).cuda()
        want = batched.plane_sum(values)
        got = torch.full((planes,), -1.0, dtype=torch.float64, device="cuda")
        assert _static_sum(values, got) == _native.HB_OK
        again = torch.full((planes,), -2.0, dtype=torch.float64, device="cuda")
        assert _static_sum(values, again) == _native.HB_OK
        torch.cuda.synchronize()
        # same kernels, same summation tree: bit-identical, and equal to numpy to rounding
        assert torch.equal(got, want) and torch.equal(again, want)
        assert np.allclose(got.cpu().numpy(), np.nansum(host.astype(np.float64), axis=1), rtol=1e-12)


def test_refuses_more_planes_than_the_scratch_holds():
    values = torch.zeros((65, 8), dtype=torch.float32, device="cuda")
    out = torch.zeros((65,), dtype=torch.float64, device="cuda")
    assert _static_sum(values, out) == _native.HB_ERR_TOO_LARGE
    assert b"64" in _native.load().hb_last_error()
    empty = torch.zeros((0, 8), dtype=torch.float32, device="cuda")
    assert _static_sum(empty, out) == _native.HB_OK
