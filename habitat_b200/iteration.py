"""Per-iteration predicted times for many training iterations at once.

The array form of what Trace.to_device(...).run_time_ms computes per trace in the
reference (analyzer/habitat/analysis/trace.py:26-51 over predictor.py:84-148):
every iteration is a list of wave-scaled kernels (one operation each, with its
launch overhead) and of MLP-predicted operations; the result is the predicted
iteration time on every destination.  Everything between the inputs and the
[iterations, destinations] totals stays on the device: the wave-scale kernel,
the fused MLP chain per operation kind, the ratio/clamp kernel and the
fixed-order float64 segment sums.
"""
from dataclasses import dataclass
from typing import Dict, Sequence

import numpy as np
import torch

from habitat_b200 import batched


@dataclass
class SpecialOps:
    """MLP-predicted operations of one kind, ordered by iteration.

    handle: batched.MLPHandle; features [n, F] float32 CUDA; run_time_ms [n]
    float32 CUDA (measured on the origin); offsets [I + 1] int64 CUDA."""
    handle: "batched.MLPHandle"
    features: torch.Tensor
    run_time_ms: torch.Tensor
    offsets: torch.Tensor


def predict_iteration_totals(kernels: batched.KernelBatch, overhead_ns: torch.Tensor,
                             kernel_offsets: torch.Tensor, special: Dict[str, SpecialOps],
                             origin, dests: Sequence, origin_mlp_row: int,
                             dest_mlp_rows: Sequence[int]):
    """-> ([I, D] float64 CUDA tensor of predicted ms per iteration and destination,
    the batched.WaveResult of the wave-scaled kernels: its scaled_ns is NaN for the pairs the
    reference would raise ZeroDivisionError on, and so are the totals of their iterations).

    A destination with the origin's name keeps the measured times, as
    MeasuredOperation.to_device does (analysis/operation.py:82-85)."""
    I = kernel_offsets.numel() - 1
    D = len(dests)
    res = batched.wave_scale(kernels, origin, dests)
    # sum over kernels of (overhead + scaled) = sum(overhead) + sum(scaled): linear, so the
    # two segment sums replace a per-kernel add
    over = batched.segment_sum(overhead_ns, kernel_offsets)                       # [I]
    measured_kernels = batched.segment_sum(kernels.run_time_ns, kernel_offsets)  # [I]
    totals = torch.empty((I, D), dtype=torch.float64, device=overhead_ns.device)
    same = [d.name == origin.name for d in dests]
    for d in range(D):
        if same[d]:
            totals[:, d] = (over + measured_kernels) / 1e6
        else:
            totals[:, d] = (over + batched.segment_sum(res.scaled_ns[d], kernel_offsets)) / 1e6
    for ops in special.values():
        n = ops.features.shape[0]
        if n == 0:
            continue
        rows = [origin_mlp_row] + [r for r, s in zip(dest_mlp_rows, same) if not s]
        T = len(rows) - 1
        measured = batched.segment_sum(ops.run_time_ms, ops.offsets)
        if T:
            feats = ops.features.repeat(T + 1, 1)
            rws = torch.tensor(rows, dtype=torch.uint8, device=feats.device).repeat_interleave(n)
            pred = ops.handle.predict(feats, rws)
            ms = batched.special_scale(ops.run_time_ms.repeat(T), pred[n:], pred[:n].repeat(T)).view(T, n)
        t = 0
        for d in range(D):
            if same[d]:
                totals[:, d] += measured
            else:
                totals[:, d] += batched.segment_sum(ms[t].contiguous(), ops.offsets)
                t += 1
    return totals, res
