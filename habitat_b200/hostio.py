"""Host-buffer pipelines: pinned host memory in, pinned host memory out.

The batched entry points in `batched.py` work on device tensors.  Callers whose
data lives on the host (the analyzer's own situation: traces and queries are
Python objects) pay two PCIe transfers per batch; these helpers keep `depth`
batches in flight on three CUDA streams (upload, compute, download) so that the
transfers of neighbouring batches overlap each other and the kernels.  Results land in pinned host tensors
owned by the pipeline; `wait(slot)` blocks until a slot's results are complete.
"""
from typing import Dict, Sequence

import torch

from habitat_b200 import batched

_VIEW = {"block_size": torch.uint16, "regs_per_thread": torch.uint16, "smem_bytes": torch.uint32}
_WAVE_OUT = ("scaled_ns", "dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves")


class _TwoStreams:
    def __init__(self, depth):
        self.depth = depth
        self.s_up = torch.cuda.Stream()
        self.s_in = torch.cuda.Stream()
        self.s_out = torch.cuda.Stream()
        self.uploaded = [torch.cuda.Event() for _ in range(depth)]
        self.computed = [torch.cuda.Event() for _ in range(depth)]
        self.downloaded = [torch.cuda.Event() for _ in range(depth)]
        self.used = [False] * depth

    def wait(self, slot):
        """Blocks the host until the results of `slot` are in its pinned buffers."""
        if self.used[slot]:
            self.downloaded[slot].synchronize()


class WaveScaleHost(_TwoStreams):
    """Wave scaling of K kernels per batch from pinned host arrays.

    submit(inputs, slot): inputs maps the six hb_kernel_soa field names to pinned
    host tensors (unsigned fields stored as their signed torch views).  Outputs
    of the batch appear in self.host_out[slot] (pinned tensors, same names as
    batched.WaveResult)."""

    def __init__(self, origin, dests: Sequence, K: int, depth: int = 2, results: Sequence[str] = _WAVE_OUT):
        """results: which outputs are copied back to the host (names of batched.WaveResult).  The
        predicted times are what the analyzer's path returns per kernel; occupancies and wave
        counts stay on the device (self.dev_out[slot]) unless they are listed."""
        super().__init__(depth)
        unknown = [r for r in results if r not in _WAVE_OUT]
        if unknown:
            raise ValueError("unknown wave-scaling outputs: %s" % unknown)
        self.origin, self.dests, self.K = origin, list(dests), K
        D = len(self.dests)
        dt = dict(num_blocks=torch.int32, block_size=torch.int16, regs_per_thread=torch.int16,
                  smem_bytes=torch.int32, run_time_ns=torch.float32, gamma=torch.float32)
        self.dev_in = [{k: torch.empty((K,), dtype=v, device="cuda") for k, v in dt.items()}
                       for _ in range(depth)]
        self.dev_out = []
        for _ in range(depth):
            self.dev_out.append(batched.WaveResult(
                scaled_ns=torch.empty((D, K), dtype=torch.float32, device="cuda"),
                dest_occupancy=torch.empty((D, K), dtype=torch.uint8, device="cuda"),
                dest_waves=torch.empty((D, K), dtype=torch.uint32, device="cuda"),
                origin_occupancy=torch.empty((K,), dtype=torch.uint8, device="cuda"),
                origin_waves=torch.empty((K,), dtype=torch.uint32, device="cuda")))
        self.host_out = [{k: torch.empty_like(getattr(o, k), device="cpu").pin_memory() for k in results}
                         for o in self.dev_out]
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in self.dev_in[0].values())
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in self.host_out[0].values())

    def submit(self, inputs: Dict[str, torch.Tensor], slot: int):
        dev = self.dev_in[slot]
        with torch.cuda.stream(self.s_up):
            # the slot's device inputs were last read by the kernel of batch (i - depth)
            if self.used[slot]:
                self.s_up.wait_event(self.computed[slot])
            for k, t in inputs.items():
                dev[k].copy_(t, non_blocking=True)
            self.uploaded[slot].record(self.s_up)
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.uploaded[slot])
            # the kernel of this batch overwrites outputs the download of batch (i - depth) reads
            if self.used[slot]:
                self.s_in.wait_event(self.downloaded[slot])
            kb = batched.KernelBatch(**{k: (t.view(_VIEW[k]) if k in _VIEW else t) for k, t in dev.items()})
            batched.wave_scale(kb, self.origin, self.dests, out=self.dev_out[slot])
            self.computed[slot].record(self.s_in)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.computed[slot])
            for k, t in self.host_out[slot].items():
                t.copy_(getattr(self.dev_out[slot], k), non_blocking=True)
            self.downloaded[slot].record(self.s_out)
        self.used[slot] = True


class MLPPredictHost(_TwoStreams):
    """MLP predictions for Q queries per batch from pinned host arrays
    (features [Q, F] float32, device rows [Q] uint8); results in self.host_out[slot]."""

    def __init__(self, handle: "batched.MLPHandle", Q: int, depth: int = 2):
        super().__init__(depth)
        self.handle, self.Q = handle, Q
        F = handle.n_op_features
        self.dev_f = [torch.empty((Q, F), dtype=torch.float32, device="cuda") for _ in range(depth)]
        self.dev_r = [torch.empty((Q,), dtype=torch.uint8, device="cuda") for _ in range(depth)]
        self.dev_o = [torch.empty((Q,), dtype=torch.float32, device="cuda") for _ in range(depth)]
        self.host_out = [torch.empty((Q,), dtype=torch.float32).pin_memory() for _ in range(depth)]
        self.h2d_bytes = Q * F * 4 + Q
        self.d2h_bytes = Q * 4

    def submit(self, features: torch.Tensor, device_rows: torch.Tensor, slot: int):
        with torch.cuda.stream(self.s_up):
            if self.used[slot]:
                self.s_up.wait_event(self.computed[slot])
            self.dev_f[slot].copy_(features, non_blocking=True)
            self.dev_r[slot].copy_(device_rows, non_blocking=True)
            self.uploaded[slot].record(self.s_up)
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.uploaded[slot])
            if self.used[slot]:
                self.s_in.wait_event(self.downloaded[slot])
            self.handle.predict(self.dev_f[slot], self.dev_r[slot], out=self.dev_o[slot])
            self.computed[slot].record(self.s_in)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.computed[slot])
            self.host_out[slot].copy_(self.dev_o[slot], non_blocking=True)
            self.downloaded[slot].record(self.s_out)
        self.used[slot] = True
