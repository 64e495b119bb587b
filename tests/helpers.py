"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

from habitat_b200 import batched, workloads
from oracle import wave as owave


def to_numpy(t):
    """CUDA tensor -> numpy, including the unsigned dtypes numpy conversion lacks."""
    t = t.detach().cpu()
    if t.dtype == torch.uint16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.uint32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.numpy()


def run_wave_gpu(kernels, origin, dests, dest_regs=None, metrics=None):
    kb = batched.KernelBatch.from_numpy(kernels)
    dr = None if dest_regs is None else torch.from_numpy(np.ascontiguousarray(dest_regs, np.int16)).cuda()
    mb = None
    if metrics is not None:
        mb = batched.KernelMetricsBatch(
            torch.from_numpy(metrics["flop_efficiency_pct"].astype(np.float64)).cuda(),
            torch.from_numpy(metrics["dram_read_bytes"].astype(np.float64)).cuda(),
            torch.from_numpy(metrics["dram_write_bytes"].astype(np.float64)).cuda(),
            torch.from_numpy(metrics["has_metrics"].astype(np.uint8)).cuda())
    res = batched.wave_scale(kb, origin, dests, dest_regs=dr, metrics=mb, want_status=True,
                             want_limits=True)
    torch.cuda.synchronize()
    out = {k: to_numpy(getattr(res, k)) for k in
           ("scaled_ns", "dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves",
            "status", "limits")}
    # the same call without the block-limit planes takes the fastest kernel the rows allow:
    # with the status plane ("fast") and without it ("plain")
    names = ("scaled_ns", "dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves")
    fast = batched.wave_scale(kb, origin, dests, dest_regs=dr, metrics=mb, want_status=True)
    torch.cuda.synchronize()
    out["fast_path"] = batched.wave_scale_path()
    out["fast"] = {k: to_numpy(getattr(fast, k)) for k in names + ("status",)}
    plain = batched.wave_scale(kb, origin, dests, dest_regs=dr, metrics=mb)
    torch.cuda.synchronize()
    out["plain_path"] = batched.wave_scale_path()
    out["plain"] = {k: to_numpy(getattr(plain, k)) for k in names}
    return out


def run_wave_oracle(kernels, origin, dests, dest_regs=None):
    specs = [origin.spec_tuple()] + [d.spec_tuple() for d in dests]
    return owave.wave_scale_batch(specs, 0, list(range(1, len(specs))), kernels, dest_regs=dest_regs)


def assert_wave_equal(got, ref, rel=1e-6):
    """Integers and status bit-exact; times within `rel` where the reference
    returns a value, NaN exactly where it raises."""
    for key in ("dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves", "status", "limits"):
        assert np.array_equal(got[key], ref[key]), key
    ok = ref["status"] <= 1
    worst = 0.0
    variants = [got] + [got[name] for name in ("fast", "plain") if name in got]
    for v in variants:
        if "status" in v:
            assert np.array_equal(v["status"], ref["status"]), "status"
        for key in ("dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves"):
            assert np.array_equal(v[key], ref[key]), key
        assert np.isnan(v["scaled_ns"][~ok]).all()
        g = v["scaled_ns"][ok].astype(np.float64)
        r = ref["scaled_ns"][ok]
        assert np.isfinite(g).all()
        if g.size:
            err = np.abs(g - r) / np.abs(r)
            assert err.max() <= rel, err.max()
            worst = max(worst, float(err.max()))
    return worst
