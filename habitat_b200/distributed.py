"""Sharding of independent kernels / queries across the GPUs of one box.

Every (kernel, destination) pair and every MLP query is independent, so ranks
take contiguous shards, run the same kernels on them and exchange nothing but
totals: one all-reduce (sums per destination) or one all-gather (per-iteration
totals) per batch, a few KB over NCCL.  The reference has no counterpart: its
prediction path is a single host thread.
"""
import ctypes
import os

import numpy as np
import torch
import torch.distributed as dist


def env_rank_world():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def init(backend=None):
    """Joins the process group described by RANK / WORLD_SIZE / MASTER_* (one
    process per GPU).  NCCL when CUDA is present, gloo otherwise."""
    rank, world = env_rank_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            local = int(os.environ.get("LOCAL_RANK", rank))
            torch.cuda.set_device(local)
            dist.init_process_group(backend, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend)
    return rank, world


_host_group = None


def host_group():
    """A gloo group over the same ranks, for waits that should not occupy the GPUs: a rank
    blocked in a NCCL barrier spins on its GPU, a rank blocked here sleeps on a socket."""
    global _host_group
    if _host_group is None and dist.is_initialized() and dist.get_world_size() > 1:
        _host_group = dist.new_group(backend="gloo")
    return _host_group


def host_barrier():
    """Barrier over the host group (no-op on one rank).  All ranks must call it."""
    g = host_group()
    if g is not None:
        dist.barrier(group=g)


def shard_bounds(n, rank, world):
    """Contiguous near-equal shards: the first n % world ranks hold one more item."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_bounds_aligned(n, rank, world, align=4):
    """As shard_bounds, but every boundary except the last is a multiple of
    `align`, so each shard keeps the wide (16-byte) load path."""
    blocks = (n + align - 1) // align
    lo, hi = shard_bounds(blocks, rank, world)
    return min(lo * align, n), min(hi * align, n)


def allreduce_sum_(totals):
    """In-place sum over ranks of a tensor of totals (no-op on one rank)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    return totals


def allgather_rows(local_rows, world=None):
    """Concatenates per-rank [n_r, D] blocks of per-iteration totals in rank order."""
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return local_rows
    world = dist.get_world_size()
    sizes = [torch.zeros(1, dtype=torch.int64, device=local_rows.device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([local_rows.shape[0]], dtype=torch.int64, device=local_rows.device))
    n_max = int(max(int(s.item()) for s in sizes))
    pad = torch.zeros((n_max,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype, device=local_rows.device)
    pad[:local_rows.shape[0]] = local_rows
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    return torch.cat([p[:int(s.item())] for p, s in zip(parts, sizes)], dim=0)


def sharded_totals(n_items, compute_totals, rank=None, world=None, align=4):
    """Runs `compute_totals(lo, hi) -> tensor of sums` on this rank's shard of
    n_items and returns the totals summed over all ranks."""
    if rank is None or world is None:
        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
    lo, hi = shard_bounds_aligned(n_items, rank, world, align)
    return allreduce_sum_(compute_totals(lo, hi))


class PeerTotals:
    """Totals summed across the GPUs of one box inside the reduction kernels themselves.

    plane_sum / group_sum work like their namesakes in `batched`, but the final stage of the
    reduction also writes its results into a mailbox on every peer GPU and adds up what the
    peers wrote (csrc/peer_exchange.cu), so the result is the sum over all ranks, identical on
    every rank, without a separate collective launch.  Create one per process after the process
    group is up (the mailbox handles travel through it); every rank must make the same calls in
    the same order on one stream.  With one rank it degenerates to the local sums."""

    def __init__(self, rank=None, world=None, connect=True):
        from habitat_b200 import _native
        self._native = _native
        lib = _native.load()
        if rank is None:
            rank = dist.get_rank() if dist.is_initialized() else 0
            world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank, self.world = rank, world
        self._handle = ctypes.c_void_p(0)
        if world == 1 or not connect:
            _native.check(lib.hb_peer_create(ctypes.byref(self._handle), rank, world))
            return
        # Every rank goes through the same collectives whether or not its own set-up worked, and
        # all ranks reach the same verdict: nobody is left waiting for a rank that gave up.
        g = host_group()
        mine, error = b"", None
        try:
            _native.check(lib.hb_peer_create(ctypes.byref(self._handle), rank, world))
            buf = (ctypes.c_uint8 * 64)()
            _native.check(lib.hb_peer_export(self._handle, buf))
            mine = bytes(buf)
        except Exception as exc:                           # noqa: BLE001 - reported to every rank below
            error = exc
        every = [None] * world
        dist.all_gather_object(every, mine, group=g)
        if all(len(b) == 64 for b in every):
            try:
                blob = (ctypes.c_uint8 * (64 * world)).from_buffer_copy(b"".join(every))
                _native.check(lib.hb_peer_connect(self._handle, blob))
            except Exception as exc:                       # noqa: BLE001
                error = exc
        verdicts = [None] * world
        dist.all_gather_object(verdicts, error is None and all(len(b) == 64 for b in every), group=g)
        if not all(verdicts):
            self.close()
            raise RuntimeError("peer exchange could not be set up on rank(s) %s%s" % (
                [r for r, v in enumerate(verdicts) if not v], ": %s" % error if error else ""))
        # every rank has mapped every mailbox before anyone writes

    def connect_local(self, others):
        """Wires up handles that live in this process on this GPU (tests: ranks walked through
        one after the other).  `others`: all PeerTotals of the group in rank order."""
        ptrs = (ctypes.c_void_p * self.world)(*[self._native.load().hb_peer_mailbox(o._handle) for o in others])
        self._native.check(self._native.load().hb_peer_connect_pointers(self._handle, ptrs))

    def plane_sum(self, values, out=None):
        """Sum over all ranks of each row of a [P, L] float32 CUDA tensor (NaN skipped) -> [P] float64."""
        P, L = values.shape
        if out is None:
            out = torch.empty((P,), dtype=torch.float64, device=values.device)
        self._native.check(self._native.load().hb_plane_sum_allreduce(
            self._handle, ctypes.c_void_p(values.data_ptr()), L, P, ctypes.c_void_p(out.data_ptr()),
            self._native.current_stream_ptr()))
        return out

    def partials_sum(self, partials, out=None):
        """Sum over all ranks of the totals a wave_scale(..., partials=) call left in `partials`
        (batched.WavePartials) -> [D] float64; a rank whose shard is empty passes partials with
        per_plane 0 and n_planes set by hand."""
        if out is None:
            out = torch.empty((partials.n_planes,), dtype=torch.float64, device=partials.buffer.device)
        self._native.check(self._native.load().hb_partials_sum_allreduce(
            self._handle, ctypes.c_void_p(partials.buffer.data_ptr()), partials.per_plane, partials.n_planes,
            ctypes.c_void_p(out.data_ptr()), self._native.current_stream_ptr()))
        return out

    def group_sum(self, values, keys, n_groups, out=None):
        """Sum over all ranks of a float32 CUDA vector grouped by a uint8 key -> [n_groups] float64."""
        if out is None:
            out = torch.empty((n_groups,), dtype=torch.float64, device=values.device)
        self._native.check(self._native.load().hb_group_sum_allreduce(
            self._handle, ctypes.c_void_p(values.data_ptr()), ctypes.c_void_p(keys.data_ptr()), values.numel(),
            n_groups, ctypes.c_void_p(out.data_ptr()), self._native.current_stream_ptr()))
        return out

    def allreduce_(self, values, phase=3):
        """In-place sum over ranks of a float64 CUDA vector of at most 64 entries."""
        self._native.check(self._native.load().hb_peer_allreduce(
            self._handle, ctypes.c_void_p(values.data_ptr()), values.numel(), phase,
            self._native.current_stream_ptr()))
        return values

    def set_wait(self, seconds):
        self._native.check(self._native.load().hb_peer_set_wait_ns(self._handle, int(seconds * 1e9)))

    def check_status(self):
        """Synchronises and raises if a wait for a peer ran out."""
        code = ctypes.c_int32(0)
        self._native.check(self._native.load().hb_peer_status(self._handle, ctypes.byref(code)))

    def close(self):
        if self._handle:
            self._native.load().hb_peer_destroy(self._handle)
            self._handle = ctypes.c_void_p(0)
