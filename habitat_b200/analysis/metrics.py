"""Kernel metrics the roofline rule reads (reference: analyzer/habitat/analysis/metrics.py).

CUPTI renamed its metrics at compute capability 7.0; a Metric knows both names
and how to bring a pre-Volta value to the post-Volta scale.
"""
from enum import Enum


class _MetricInfo:
    def __init__(self, cupti_name, legacy_cupti_name, legacy_to_canonical_fn):
        self._cupti_name = cupti_name
        self._legacy_cupti_name = legacy_cupti_name
        self._legacy_to_canonical_fn = legacy_to_canonical_fn

    @property
    def cupti_name(self):
        return self._cupti_name

    @property
    def legacy_cupti_name(self):
        return self._legacy_cupti_name

    def to_canonical_value(self, value, device):
        return value if device.compute_capability[0] >= 7 else self._legacy_to_canonical_fn(value)


def _same(value):
    return value


class Metric(Enum):
    DRAMUtilization = _MetricInfo(
        "dram__throughput.avg.pct_of_peak_sustained_elapsed", "dram_utilization", lambda v: v * 10)
    DRAMReadBytes = _MetricInfo("dram__bytes_read.sum", "dram_read_bytes", _same)
    DRAMWriteBytes = _MetricInfo("dram__bytes_write.sum", "dram_write_bytes", _same)
    SinglePrecisionFLOPEfficiency = _MetricInfo(
        "smsp__sass_thread_inst_executed_ops_fadd_fmul_ffma_pred_on.avg.pct_of_peak_sustained_elapsed",
        "flop_sp_efficiency", _same)
    SinglePrecisionAddOps = _MetricInfo(
        "smsp__sass_thread_inst_executed_op_fadd_pred_on.sum", "flop_count_sp_add", _same)


def _metric_name(metric, device):
    if not isinstance(metric, Metric):
        return metric  # already a raw CUPTI string
    info = metric.value
    return info.cupti_name if device.compute_capability[0] >= 7 else info.legacy_cupti_name


def resolve_metrics(metrics, device):
    """Metric values -> the raw CUPTI names valid on `device` (a new list)."""
    if metrics is None:
        return []
    if isinstance(metrics, (list, tuple)):
        return [_metric_name(m, device) for m in metrics]
    return [_metric_name(metrics, device)]
