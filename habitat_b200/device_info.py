"""A device-table row for the GPU in this machine.

Does what two offline tools of the reference do together: `habitat-device-info`
(cpp/src/device_info.cpp:16-30) prints the occupancy fields of a devices.yml row, and
tools/device-metadata/measure_peak_flops.py estimates peak_gflops_per_second.  Here both come
from the native library (hb_device_info, hb_peak_flops_test); the peak is what a fused
multiply-add kernel achieves, not a profiler-derived estimate.

    python -m habitat_b200.device_info [--device 0] [--name B200] [--trials 5]

prints the row in the reference's one-mapping-per-device YAML form.
"""
import argparse
import ctypes

from habitat_b200 import _native
from habitat_b200.habitat_cuda import DeviceProperties


def query_device(device=0, name=None, measure_peak=False, trials=5):
    """DeviceProperties of CUDA device `device`.  With measure_peak the single-precision
    peak is the measured one (the device must be the current one), else the nominal
    FMA lanes x SMs x clock."""
    lib = _native.load()
    spec = _native.DeviceSpec()
    _native.check(lib.hb_device_info(int(device), ctypes.byref(spec)))
    fields = {f: int(getattr(spec, f)) for f in _native.DEVICE_SPEC_FIELDS}
    if measure_peak:
        fields["peak_gflops_per_second"] = int(round(measure_peak_gflops(device, trials)))
    if name is None:
        import torch
        name = "".join(c if c.isalnum() else "_" for c in torch.cuda.get_device_name(device))
    return DeviceProperties(name=name, **fields)


def measure_peak_gflops(device=0, trials=5):
    """Best achieved fp32 GFLOP/s of the FMA probe kernel over `trials` launches."""
    import torch
    lib = _native.load()
    out = ctypes.c_double(0.0)
    with torch.cuda.device(device):
        _native.check(lib.hb_peak_flops_test(int(trials), ctypes.byref(out), _native.current_stream_ptr()))
    return float(out.value)


def as_yaml(props):
    """The row as the reference's devices.yml writes it (plus the reserved shared memory)."""
    fields = dict(zip(_native.DEVICE_SPEC_FIELDS, props.spec_tuple()))
    lines = ["%s:" % props.name]
    lines += ["  %s: %d" % (k, v) for k, v in fields.items()]
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser(description="Print a device-table row for a GPU of this machine.")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--name", default=None)
    ap.add_argument("--trials", type=int, default=5)
    ap.add_argument("--nominal-peak", action="store_true",
                    help="do not run the FMA probe; report FMA lanes x SMs x clock")
    args = ap.parse_args(argv)
    print(as_yaml(query_device(args.device, args.name, measure_peak=not args.nominal_peak,
                               trials=args.trials)))


if __name__ == "__main__":
    main()
