"""Host-buffer pipelines: pinned host memory in, pinned host memory out.

The batched entry points in `batched.py` work on device tensors.  Callers whose
data lives on the host (the analyzer's own situation: traces and queries are
Python objects) pay two PCIe transfers per batch; these helpers keep `depth`
batches in flight on three CUDA streams (upload, compute, download) so that the
transfers of neighbouring batches overlap each other and the kernels.  A batch
travels as ONE contiguous block each way (one copy up, one copy down): the six
record fields are laid out back to back in a pinned block (`pack_kernels`), the
device keeps a block of the same layout per slot and the kernel reads typed
views of it.  Results land in pinned host tensors owned by the pipeline;
`wait(slot)` blocks until a slot's results are complete.
"""
import contextlib
import os
from typing import Sequence

import numpy as np
import torch

from habitat_b200 import batched

# field order inside a record block: the 4-byte fields first, so that every field starts on an
# 8-byte boundary whenever K is even
_FIELDS = (("num_blocks", torch.int32, 4), ("run_time_ns", torch.float32, 4), ("gamma", torch.float32, 4),
           ("smem_bytes", torch.uint32, 4), ("block_size", torch.uint16, 2), ("regs_per_thread", torch.uint16, 2))
RECORD_BYTES = sum(size for _, _, size in _FIELDS)      # 20
_WAVE_OUT = ("scaled_ns", "dest_occupancy", "dest_waves", "origin_occupancy", "origin_waves")


def _views(block: torch.Tensor, K: int):
    """Typed views of a [K * 20] uint8 block, by field name."""
    out, at = {}, 0
    for name, dtype, size in _FIELDS:
        out[name] = block[at:at + K * size].view(dtype)
        at += K * size
    return out


def pack_kernels(arrays, out: torch.Tensor = None) -> torch.Tensor:
    """The six record fields of `arrays` (numpy, as workloads.make_kernels returns them) laid
    out back to back in one pinned uint8 block of K * 20 bytes."""
    K = len(arrays["num_blocks"])
    if out is None:
        out = torch.empty((K * RECORD_BYTES,), dtype=torch.uint8).pin_memory()
    host = out.numpy()
    at = 0
    np_dt = {"num_blocks": np.int32, "run_time_ns": np.float32, "gamma": np.float32, "smem_bytes": np.uint32,
             "block_size": np.uint16, "regs_per_thread": np.uint16}
    for name, _, size in _FIELDS:
        host[at:at + K * size] = np.ascontiguousarray(arrays[name]).astype(np_dt[name], copy=False).view(np.uint8)
        at += K * size
    return out


def gpu_numa_cpus(gpu_index: int):
    """CPUs of the NUMA node the GPU hangs off (from sysfs), or None when that cannot be told."""
    try:
        bus = torch.cuda.get_device_properties(gpu_index).pci_bus_id
        dom = torch.cuda.get_device_properties(gpu_index).pci_domain_id
        dev = torch.cuda.get_device_properties(gpu_index).pci_device_id
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/numa_node" % (dom, bus, dev)
        node = int(open(path).read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        return cpus & os.sched_getaffinity(0) or None
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


@contextlib.contextmanager
def numa_local(gpu_index: int):
    """Runs the enclosed allocations on a CPU of the GPU's NUMA node, so that pinned pages are
    placed (first touch) in the memory closest to the GPU's PCIe root.  A no-op when the
    topology cannot be read."""
    cpus = gpu_numa_cpus(gpu_index)
    before = os.sched_getaffinity(0)
    if cpus:
        os.sched_setaffinity(0, cpus)
    try:
        yield cpus
    finally:
        if cpus:
            os.sched_setaffinity(0, before)


class _Streams:
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


class WaveScaleHost(_Streams):
    """Wave scaling of K kernels per batch from pinned host blocks.

    submit(block, slot): `block` is a pinned uint8 tensor from pack_kernels (K * 20 bytes).
    The outputs listed in `results` appear in self.host_out[slot] (pinned tensors, same names
    as batched.WaveResult); the predicted times are what the analyzer's path returns per
    kernel, the other outputs stay on the device (self.dev_out[slot]) unless listed.
    "totals" asks for the [D] float64 per-destination sums of the batch's predicted times (what
    Trace.run_time_ms is per destination): the kernel's blocks add up their own results, so a
    caller that only wants totals (results=("totals",)) downloads 8 D bytes per batch."""

    def __init__(self, origin, dests: Sequence, K: int, depth: int = 3, results: Sequence[str] = ("scaled_ns",)):
        super().__init__(depth)
        unknown = [r for r in results if r not in _WAVE_OUT + ("totals",)]
        if unknown:
            raise ValueError("unknown wave-scaling outputs: %s" % unknown)
        self.origin, self.dests, self.K = origin, list(dests), K
        D = len(self.dests)
        self.want_totals = "totals" in results
        results = [r for r in results if r != "totals"]
        if self.want_totals:
            self.partials = [batched.WavePartials(K, D) for _ in range(depth)]
            self.dev_totals = [torch.zeros((D,), dtype=torch.float64, device="cuda") for _ in range(depth)]
        self.dev_block = [torch.empty((K * RECORD_BYTES,), dtype=torch.uint8, device="cuda") for _ in range(depth)]
        self.dev_in = [batched.KernelBatch(**_views(b, K)) for b in self.dev_block]
        self.dev_out = []
        for _ in range(depth):
            self.dev_out.append(batched.WaveResult(
                scaled_ns=torch.empty((D, K), dtype=torch.float32, device="cuda"),
                dest_occupancy=torch.empty((D, K), dtype=torch.uint8, device="cuda"),
                dest_waves=torch.empty((D, K), dtype=torch.uint32, device="cuda"),
                origin_occupancy=torch.empty((K,), dtype=torch.uint8, device="cuda"),
                origin_waves=torch.empty((K,), dtype=torch.uint32, device="cuda")))
        with numa_local(torch.cuda.current_device()):
            self.host_out = [{k: torch.empty_like(getattr(o, k), device="cpu").pin_memory() for k in results}
                             for o in self.dev_out]
            if self.want_totals:
                for h in self.host_out:
                    h["totals"] = torch.zeros((D,), dtype=torch.float64).pin_memory()
        self.h2d_bytes = K * RECORD_BYTES
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in self.host_out[0].values())

    def submit(self, block: torch.Tensor, slot: int):
        if block.numel() != self.K * RECORD_BYTES or block.dtype != torch.uint8:
            raise ValueError("block must be a uint8 tensor of K * %d bytes (pack_kernels)" % RECORD_BYTES)
        with torch.cuda.stream(self.s_up):
            # the slot's device inputs were last read by the kernel of batch (i - depth)
            if self.used[slot]:
                self.s_up.wait_event(self.computed[slot])
            self.dev_block[slot].copy_(block, non_blocking=True)
            self.uploaded[slot].record(self.s_up)
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.uploaded[slot])
            # the kernel of this batch overwrites outputs the download of batch (i - depth) reads
            if self.used[slot]:
                self.s_in.wait_event(self.downloaded[slot])
            if self.want_totals:
                batched.wave_scale(self.dev_in[slot], self.origin, self.dests, out=self.dev_out[slot],
                                   partials=self.partials[slot])
                self.partials[slot].totals(out=self.dev_totals[slot])
            else:
                batched.wave_scale(self.dev_in[slot], self.origin, self.dests, out=self.dev_out[slot])
            self.computed[slot].record(self.s_in)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.computed[slot])
            for k, t in self.host_out[slot].items():
                t.copy_(self.dev_totals[slot] if k == "totals" else getattr(self.dev_out[slot], k), non_blocking=True)
            self.downloaded[slot].record(self.s_out)
        self.used[slot] = True


class MLPPredictHost(_Streams):
    """MLP predictions for up to Q queries per batch from pinned host arrays
    (features [q, F] float32, device rows [q] uint8, q <= Q); results in self.host_out[slot][:q]."""

    def __init__(self, n_op_features: int, Q: int, depth: int = 3):
        super().__init__(depth)
        self.Q, F = Q, n_op_features
        self.dev_f = [torch.empty((Q, F), dtype=torch.float32, device="cuda") for _ in range(depth)]
        self.dev_r = [torch.empty((Q,), dtype=torch.uint8, device="cuda") for _ in range(depth)]
        self.dev_o = [torch.empty((Q,), dtype=torch.float32, device="cuda") for _ in range(depth)]
        with numa_local(torch.cuda.current_device()):
            self.host_out = [torch.empty((Q,), dtype=torch.float32).pin_memory() for _ in range(depth)]
        self.h2d_bytes = Q * F * 4 + Q
        self.d2h_bytes = Q * 4

    def submit(self, handle: "batched.MLPHandle", features: torch.Tensor, device_rows: torch.Tensor, slot: int):
        q = features.shape[0]
        if q > self.Q or features.shape[1] != self.dev_f[slot].shape[1]:
            raise ValueError("batch does not fit the pipeline's buffers")
        with torch.cuda.stream(self.s_up):
            if self.used[slot]:
                self.s_up.wait_event(self.computed[slot])
            self.dev_f[slot][:q].copy_(features, non_blocking=True)
            self.dev_r[slot][:q].copy_(device_rows, non_blocking=True)
            self.uploaded[slot].record(self.s_up)
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.uploaded[slot])
            if self.used[slot]:
                self.s_in.wait_event(self.downloaded[slot])
            handle.predict(self.dev_f[slot][:q], self.dev_r[slot][:q], out=self.dev_o[slot][:q])
            self.computed[slot].record(self.s_in)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.computed[slot])
            self.host_out[slot][:q].copy_(self.dev_o[slot][:q], non_blocking=True)
            self.downloaded[slot].record(self.s_out)
        self.used[slot] = True
