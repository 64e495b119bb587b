"""Measured and predicted kernels (reference: analyzer/habitat/analysis/kernels.py)."""


class MeasuredKernel:
    """A recorded kernel: timing record plus the records that carry its metrics."""

    def __init__(self, time_kernel, metrics_kernels, device):
        self._c = time_kernel
        self._metrics_kernels = metrics_kernels
        self._device = device
        self._cached_metrics = {}

    def get_metric(self, metric_info, default=None):
        """Canonical value of a Metric; AttributeError if absent and no default."""
        if metric_info in self._cached_metrics:
            return self._cached_metrics[metric_info]
        info = metric_info.value
        for record in self._metrics_kernels:
            for raw_name, raw_value in record.metrics:
                if raw_name in (info.cupti_name, info.legacy_cupti_name):
                    value = info.to_canonical_value(raw_value, self._device)
                    self._cached_metrics[metric_info] = value
                    return value
        if default is None:
            raise AttributeError("Unknown metric: {}".format(metric_info.name))
        return default

    def __getattr__(self, name):
        # everything else (name, num_blocks, run_time_ns, thread_block_occupancy, ...)
        # is answered by the underlying KernelInstance
        return getattr(self._c, name)


class PredictedKernel:
    def __init__(self, measured_kernel, run_time_ns):
        self._measured_kernel = measured_kernel
        self._run_time_ns = run_time_ns

    @property
    def run_time_ns(self):
        return self._run_time_ns

    @property
    def name(self):
        return self._measured_kernel.name
