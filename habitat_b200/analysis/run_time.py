"""Run times of one pass of an operation (reference: analyzer/habitat/analysis/run_time.py)."""
from habitat_b200.utils import ns_to_ms


class RunTime:
    @property
    def run_time_ms(self):
        raise NotImplementedError

    @property
    def ktime_ns(self):
        return sum(k.run_time_ns for k in self.kernels)

    @property
    def kernels(self):
        return []

    @property
    def device(self):
        raise NotImplementedError


class RunTimeMeasurement(RunTime):
    """Measured wall time of a pass and the kernels recorded in it."""

    def __init__(self, run_time_ms, kernels, device):
        self._run_time_ms = run_time_ms
        self._kernels = kernels
        self._device = device

    @property
    def run_time_ms(self):
        return self._run_time_ms

    @property
    def kernels(self):
        return self._kernels

    @property
    def device(self):
        return self._device


class RunTimePrediction(RunTime):
    """Predicted kernels plus the launch overhead carried over unchanged."""

    def __init__(self, overhead_ns, predicted_kernels, device):
        self._overhead_ns = overhead_ns
        self._predicted_kernels = predicted_kernels
        self._device = device
        self._run_time_ms = None

    @property
    def run_time_ms(self):
        if self._run_time_ms is None:
            total_ns = self._overhead_ns + sum(k.run_time_ns for k in self._predicted_kernels)
            self._run_time_ms = ns_to_ms(total_ns)
        return self._run_time_ms

    @property
    def kernels(self):
        return self._predicted_kernels

    @property
    def device(self):
        return self._device


class RunTimePurePrediction(RunTime):
    """A predicted time with no kernel breakdown (MLP-predicted operations)."""

    def __init__(self, run_time_ms, device):
        if run_time_ms is None:
            # the reference would fail later, on an attribute it never sets
            # (run_time.py:76-83); refuse at construction instead
            raise ValueError("RunTimePurePrediction needs a run time")
        self._run_time_ms = run_time_ms
        self._device = device

    @property
    def run_time_ms(self):
        return self._run_time_ms

    @property
    def device(self):
        return self._device
