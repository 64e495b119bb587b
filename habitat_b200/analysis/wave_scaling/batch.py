"""Flattening of recorded kernels into the structure-of-arrays the device path takes.

This is the host half of wave scaling: it walks MeasuredKernel objects once,
resolves metrics and per-destination register counts, and hands flat arrays to
the fused kernel (habitat_b200/csrc/wave_scale.cu).  No scaling arithmetic
happens here.
"""
import numpy as np
import torch

from habitat_b200 import batched
from habitat_b200.analysis.metrics import Metric

ROOFLINE, RESIMPLIFIED, UNIFIED = "roofline", "resimplified", "unified"

_NEEDED = (Metric.SinglePrecisionFLOPEfficiency, Metric.DRAMReadBytes, Metric.DRAMWriteBytes)


def flatten_kernels(kernels, mode):
    """kernels: sequence of MeasuredKernel (or objects with the same surface).
    Returns (arrays, metrics or None, names)."""
    K = len(kernels)
    nb = np.empty(K, np.int32)
    bs = np.empty(K, np.uint16)
    rg = np.empty(K, np.uint16)
    sm = np.empty(K, np.uint32)
    tm = np.empty(K, np.float64)
    eff = np.zeros(K, np.float64)
    rd = np.zeros(K, np.float64)
    wr = np.zeros(K, np.float64)
    has = np.zeros(K, np.uint8)
    names = []
    for i, k in enumerate(kernels):
        record = getattr(getattr(k, "_c", k), "launch_record", None)
        if record is not None:
            name, blocks, block_size, regs, smem, time_ns = record()
        else:
            # any object with the reference's KernelInstance surface
            md = k.metadata
            name, blocks, time_ns = k.name, k.num_blocks, k.run_time_ns
            block_size, regs = int(md["block_size"]), int(md["registers_per_thread"])
            smem = int(md["static_shared_memory"]) + int(md["dynamic_shared_memory"])
        nb[i] = blocks
        bs[i] = min(max(block_size, 0), 0xFFFF)
        rg[i] = regs & 0xFFFF
        sm[i] = smem if 0 <= smem <= 0xFFFFFFFF else 0xFFFFFFFF
        tm[i] = time_ns
        names.append(name)
        if mode != RESIMPLIFIED:
            if getattr(k, "_metrics_kernels", None) == [] and not k._cached_metrics:
                # no metric records at all: the look-up below could only raise
                if mode == ROOFLINE:
                    raise AttributeError("Unknown metric: {}".format(_NEEDED[0].name))
                continue
            try:
                vals = [k.get_metric(m) for m in _NEEDED]
            except AttributeError:
                if mode == ROOFLINE:
                    raise
                continue
            eff[i], rd[i], wr[i] = vals
            has[i] = 1
    arrays = dict(num_blocks=nb, block_size=bs, regs_per_thread=rg, smem_bytes=sm, run_time_ns=tm,
                  gamma=np.ones(K, np.float32))
    metrics = None
    if mode != RESIMPLIFIED and has.any():
        metrics = dict(flop_efficiency_pct=eff, dram_read_bytes=rd, dram_write_bytes=wr,
                       has_metrics=has)
    return arrays, metrics, names


class FlatKernels:
    """The kernels of a trace flattened once and resident on the GPU: what a repeated
    prediction of the same trace (other destinations, another strategy argument) reuses
    instead of walking the kernel objects again."""

    def __init__(self, kernels, mode):
        arrays, metrics, self.names = flatten_kernels(kernels, mode)
        self.mode = mode
        self.count = len(kernels)
        self.batch = batched.KernelBatch.from_numpy(arrays)
        self.metrics = None
        if metrics is not None:
            self.metrics = batched.KernelMetricsBatch(
                torch.from_numpy(metrics["flop_efficiency_pct"]).cuda(),
                torch.from_numpy(metrics["dram_read_bytes"]).cuda(),
                torch.from_numpy(metrics["dram_write_bytes"]).cuda(),
                torch.from_numpy(metrics["has_metrics"]).cuda())


def scale_kernels(kernels, origin_device, dest_devices, metadata_manager, mode=UNIFIED, flat=None):
    """Runs the fused kernel for `kernels` x `dest_devices`.

    `flat` is a FlatKernels of the same kernels and mode from an earlier call (or None).
    Returns a WaveResult whose tensors live on the GPU; nothing is synchronised here."""
    if flat is None or flat.mode != mode or flat.count != len(kernels):
        flat = FlatKernels(kernels, mode)
    kb, mb, names = flat.batch, flat.metrics, flat.names
    dest_regs = None
    if metadata_manager is not None and hasattr(metadata_manager, "registers_matrix"):
        m = metadata_manager.registers_matrix(names, dest_devices)
        if m is not None:
            dest_regs = torch.from_numpy(m).cuda()
    elif metadata_manager is not None:
        # a foreign manager with only the per-kernel query of the reference
        m = np.full((len(dest_devices), len(kernels)), -1, np.int16)
        for d, dev in enumerate(dest_devices):
            for i, k in enumerate(kernels):
                r = metadata_manager.kernel_registers_for(k, dev)
                if r is not None:
                    m[d, i] = r
        if (m >= 0).any():
            dest_regs = torch.from_numpy(m).cuda()
    return batched.wave_scale(kb, origin_device, dest_devices, dest_regs=dest_regs, metrics=mb)


def raise_like_reference(scaled_ns_host):
    """The reference divides by a zero wave size for the pairs whose predicted time the
    kernel leaves as NaN (roofline.py:29-45: a kernel the origin cannot run at all, or one
    that fits in an origin wave going to a device that cannot run it)."""
    if np.isnan(scaled_ns_host).any():
        raise ZeroDivisionError("integer division or modulo by zero")
