"""Cross-device prediction of operations and whole traces.

Reference: analyzer/habitat/analysis/predictor.py.  Same constructor, the same
four predictor attributes and the same predict_operation(); what differs is the
inside: instead of one Python call per kernel and two CPU forwards per special
operation, a trace is flattened once and goes through three device launches
(wave scaling, the fused MLP chain per operation kind, the ratio/clamp), for
any number of destination devices at a time (predict_trace).
"""
import collections.abc
import functools
import logging
import operator
import os

import numpy as np
import torch

from habitat_b200 import batched
from habitat_b200.analysis import SPECIAL_OPERATIONS
from habitat_b200.analysis.kernels import PredictedKernel
from habitat_b200.analysis.mlp.mlp import RuntimePredictor
from habitat_b200.analysis.operation import PredictedOperation
from habitat_b200.analysis.run_time import RunTimePrediction, RunTimePurePrediction
from habitat_b200.analysis.wave_scaling import batch as wave_batch
from habitat_b200.analysis.wave_scaling.metadata import MetadataManager
from habitat_b200.analysis.wave_scaling.unified import unified_wave_scaling
from habitat_b200.data import path_to_data
from habitat_b200.utils import name_all_arguments

logger = logging.getLogger(__name__)

# positional parameter names of the torch callables whose arguments were recorded
CONV2D_PARAMS = ["input", "weight", "bias", "stride", "padding", "dilation", "groups"]
LINEAR_PARAMS = ["input", "weight", "bias"]
BMM_PARAMS = ["input", "mat2", "out"]
LSTM_PARAMS_NO_BATCH_SIZES = ["input", "hx", "flat_weights", "bias", "num_layers", "dropout",
                              "training", "bidirectional", "batch_first"]
LSTM_PARAMS = ["input", "batch_sizes", "hx", "flat_weights", "bias", "num_layers", "dropout",
               "training", "bidirectional"]
MATMUL_PARAMS = ["input", "other", "out"]

_MLP_OPS = ("conv2d", "lstm", "linear", "bmm")


def _first(value):
    return value[0] if isinstance(value, tuple) else value


def conv2d_features(operation):
    """predictor.py:150-176 of the reference."""
    a = name_all_arguments(CONV2D_PARAMS, operation.arguments.args, operation.arguments.kwargs)
    return dict(batch=a["input"][0], image_size=a["input"][2], in_channels=a["input"][1],
                out_channels=a["weight"][0], kernel_size=a["weight"][2], stride=_first(a["stride"]),
                padding=_first(a["padding"]), bias=0 if a["bias"] is None else 1)


def linear_features(operation):
    """predictor.py:184-213: every leading input dimension counts towards the batch."""
    a = name_all_arguments(LINEAR_PARAMS, operation.arguments.args, operation.arguments.kwargs)
    return dict(batch=functools.reduce(operator.mul, a["input"][:-1]), in_features=a["weight"][1],
                out_features=a["weight"][0], bias=0 if a["bias"] is None else 1)


def bmm_features(operation):
    """predictor.py:220-232."""
    a = name_all_arguments(BMM_PARAMS, operation.arguments.args, operation.arguments.kwargs)
    return dict(batch=a["input"][0], left=a["input"][1], middle=a["input"][2], right=a["mat2"][2])


def lstm_features(operation):
    """predictor.py:240-277: the two torch LSTM overloads are told apart by the
    type of the fifth positional argument."""
    args, kwargs = operation.arguments.args, operation.arguments.kwargs
    if not isinstance(args[4], bool):
        a = name_all_arguments(LSTM_PARAMS_NO_BATCH_SIZES, args, kwargs)
        batch, seq_len, input_size = a["input"][1], a["input"][0], a["input"][2]
    else:
        a = name_all_arguments(LSTM_PARAMS, args, kwargs)
        batch = max(operation.arguments.special["batch_sizes"])
        seq_len, input_size = a["input"][0] // batch, a["input"][1]
    return dict(bias=0 if a["bias"] is None else 1, bidirectional=1 if a["bidirectional"] else 0,
                batch=batch, seq_len=seq_len, input_size=input_size, hidden_size=a["hx"][0][2],
                num_layers=a["num_layers"])


_EXTRACTORS = {"conv2d": conv2d_features, "linear": linear_features, "bmm": bmm_features,
               "lstm": lstm_features}


# Batched form of the extractors above for the common recording (every argument positional,
# as torch passes them): one tuple per operation, no dictionaries.  Operations recorded with
# keyword arguments, and the LSTM overloads, go through the named path.
def _conv2d_row(a):
    x, w = a[0], a[1]
    return (x[0], x[2], x[1], w[0], w[2], _first(a[3]), _first(a[4]), 0 if a[2] is None else 1)


def _linear_row(a):
    x, w = a[0], a[1]
    batch = 1
    for v in x[:-1]:
        batch *= v
    return (batch, w[1], w[0], 0 if a[2] is None else 1)


def _bmm_row(a):
    x = a[0]
    return (x[0], x[1], x[2], a[1][2])


_FAST_ROWS = {
    "conv2d": (_conv2d_row, 5, ("batch", "image_size", "in_channels", "out_channels", "kernel_size",
                                "stride", "padding", "bias")),
    "linear": (_linear_row, 3, ("batch", "in_features", "out_features", "bias")),
    "bmm": (_bmm_row, 2, ("batch", "left", "middle", "right")),
}


def feature_matrix(name, operations, order):
    """[n, F] float32 features of `operations` (all of kind `name`) in the column order `order`."""
    fast = _FAST_ROWS.get(name)
    if fast is not None:
        row, arity, columns = fast
        try:
            rows = [row(op.arguments.args) if len(op.arguments.args) >= arity and not op.arguments.kwargs
                    else None for op in operations]
        except (TypeError, IndexError):
            rows = [None]
        if None not in rows:
            m = np.array(rows, dtype=np.float32).reshape(len(rows), len(columns))
            return np.ascontiguousarray(m[:, [columns.index(f) for f in order]])
    extract = _EXTRACTORS[name]
    return np.array([[extract(op)[f] for f in order] for op in operations], dtype=np.float32)


class _LazyRunTimePrediction(RunTimePrediction):
    """A predicted pass whose time is known (summed on the device) and whose
    PredictedKernel objects are only built when somebody asks for them."""

    def __init__(self, overhead_ns, measured_kernels, times_ns, total_kernel_ns, device):
        super().__init__(overhead_ns=overhead_ns, predicted_kernels=None, device=device)
        self._measured_kernels = measured_kernels
        self._times_ns = times_ns
        self._run_time_ms = (overhead_ns + total_kernel_ns) / 1e6

    @property
    def kernels(self):
        if self._predicted_kernels is None:
            self._predicted_kernels = [PredictedKernel(k, float(t))
                                       for k, t in zip(self._measured_kernels, self._times_ns)]
        return self._predicted_kernels


class _GroupPlan:
    """Everything about the operations of one origin device that does not depend on the
    destination: which operation is predicted how, the flattened kernels of the wave-scaled
    passes, launch overheads, MLP feature matrices.  Built by the first prediction of a trace
    and kept with it."""

    def __init__(self, operations, indices, mode):
        self.indices = np.asarray(indices, np.int64)
        self.mode = mode
        wave_idx, fwd_run, bwd_run, runs = [], [], [], []
        self.mlp_idx = {op: [] for op in _MLP_OPS}
        self.passthrough_idx = []
        for i in indices:
            op = operations[i]
            name = op.name
            if name not in SPECIAL_OPERATIONS:
                wave_idx.append(i)
                fwd_run.append(len(runs))
                runs.append(op.forward)
                if op.backward is not None:
                    bwd_run.append(len(runs))
                    runs.append(op.backward)
                else:
                    bwd_run.append(-1)
            elif name in self.mlp_idx:
                self.mlp_idx[name].append(i)
            else:
                logger.warning("Unhandled special operation: %s", name)
                self.passthrough_idx.append(i)
        self.wave_idx = np.asarray(wave_idx, np.int64)
        self.fwd_run = np.asarray(fwd_run, np.int64)
        self.bwd_run = np.asarray(bwd_run, np.int64)
        self.runs = runs
        self.kernels = []
        offsets = [0]
        for run in runs:
            self.kernels.extend(run.kernels)
            offsets.append(len(self.kernels))
        self.offsets = np.asarray(offsets, np.int64)
        self.flat = wave_batch.FlatKernels(self.kernels, mode) if (self.kernels and mode is not None) else None
        # launch overhead of a pass (predictor.py:113-116 of the reference): wall time minus kernel time
        measured = np.array([k.run_time_ns for k in self.kernels], np.float64)
        per_run = np.add.reduceat(np.concatenate([measured, [0.0]]), self.offsets[:-1]) if runs else np.zeros(0)
        per_run = np.where(self.offsets[1:] > self.offsets[:-1], per_run, 0.0) if runs else per_run
        wall_ns = np.array([run.run_time_ms for run in runs], np.float64) * 1e6
        self.overheads = np.maximum(wall_ns - per_run, 0.0)
        self.offsets_dev = None
        self.mlp_inputs = {}      # op kind -> (feature matrix, measured ms), filled on first use


class PredictedOperations(collections.abc.Sequence):
    """The operations of a trace as predicted for one destination.  Behaves like the list the
    reference builds (len, indexing, iteration); PredictedOperation, RunTimePrediction and
    PredictedKernel objects are created when an element is first touched, the per-operation
    times (`run_times_ms`) and their sum (`total_run_time_ms`) are there from the start."""

    def __init__(self, operations, dest):
        self._operations = operations
        self._dest = dest
        n = len(operations)
        self._made = [None] * n
        self._kind = np.zeros(n, np.int8)       # 0 as measured, 1 wave-scaled, 2 MLP, 3 special passed through
        self._group = np.zeros(n, np.int32)
        self._a = np.full(n, -1, np.int64)      # wave: forward run; MLP: position in the group's ms array
        self._b = np.full(n, -1, np.int64)      # wave: backward run or -1
        self._groups = []                       # per origin group: dict(plan, times, totals, ms)
        self.run_times_ms = np.zeros(n, np.float64)
        self._total = None

    def __len__(self):
        return len(self._operations)

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[j] for j in range(*i.indices(len(self)))]
        if i < 0:
            i += len(self)
        made = self._made[i]
        if made is None:
            made = self._made[i] = self._make(i)
        return made

    @property
    def total_run_time_ms(self):
        if self._total is None:
            self._total = float(self.run_times_ms.sum())
        return self._total

    def _make(self, i):
        op = self._operations[i]
        kind = self._kind[i]
        if kind == 0:
            return op
        if kind == 3:
            return PredictedOperation(op, op.forward, op.backward, self._dest)
        g = self._groups[self._group[i]]
        if kind == 2:
            return PredictedOperation(op, RunTimePurePrediction(float(self.run_times_ms[i]), self._dest),
                                      None, self._dest)
        plan = g["plan"]

        def run(r):
            lo, hi = plan.offsets[r], plan.offsets[r + 1]
            return _LazyRunTimePrediction(float(plan.overheads[r]), plan.kernels[lo:hi], g["times"][lo:hi],
                                          float(g["totals"][r]), self._dest)
        b = self._b[i]
        return PredictedOperation(op, run(self._a[i]), run(b) if b >= 0 else None, self._dest)


class Predictor:
    def __init__(self, kernel_metadata_file=None, wave_scaling_strategy=unified_wave_scaling, *,
                 model_paths=None, precision=None):
        if kernel_metadata_file is None:
            default = path_to_data("kernels.sqlite")
            kernel_metadata_file = default if os.path.exists(default) else None
        self._kernel_metadata = MetadataManager(kernel_metadata_file)
        self._wave_scaling_strategy = wave_scaling_strategy
        # "bf16" (2e-2 relative against the float32 reference) or "bf16x3" (1e-4); the environment
        # variable HABITAT_B200_PRECISION chooses for callers that keep the reference's constructor call
        self._precision = precision or os.environ.get("HABITAT_B200_PRECISION", "bf16")
        if self._precision not in ("bf16", "bf16x3"):
            raise ValueError("precision must be 'bf16' or 'bf16x3', got %r" % (self._precision,))
        self._model_paths = dict(model_paths or {})
        self._predictors = {}

    # The four predictors load on first use: their checkpoints are large and,
    # unlike the reference, most traces do not need all of them.
    def _predictor(self, op):
        if op not in self._predictors:
            path = self._model_paths.get(op, path_to_data("%s/model.pth" % op))
            if not os.path.exists(path):
                raise FileNotFoundError(
                    "no checkpoint for the %s predictor at %s (pass model_paths= or assign "
                    "Predictor.%s_pred)" % (op, path, op))
            self._predictors[op] = RuntimePredictor(op, 8, 1024, path, precision=self._precision)
        return self._predictors[op]

    linear_pred = property(lambda self: self._predictor("linear"),
                           lambda self, v: self._predictors.__setitem__("linear", v))
    lstm_pred = property(lambda self: self._predictor("lstm"),
                         lambda self, v: self._predictors.__setitem__("lstm", v))
    conv2d_pred = property(lambda self: self._predictor("conv2d"),
                           lambda self, v: self._predictors.__setitem__("conv2d", v))
    bmm_pred = property(lambda self: self._predictor("bmm"),
                        lambda self, v: self._predictors.__setitem__("bmm", v))

    # ------------------------------------------------------------------
    def predict_operation(self, operation, dest_device):
        return self.predict_trace([operation], [dest_device])[0][0]

    def predict_trace(self, operations, dest_devices, cache=None):
        """Predicts every operation on every destination.

        Returns one sequence of operations per destination, in order (PredictedOperations:
        list-like, elements built on first access); operations measured on a device of the
        same name as the destination are returned as they are (analysis/trace.py:40-41 and
        operation.py:82-85).  `cache` is a dict the caller keeps with the operations (Trace
        does): the destination-independent plan of the trace (flattened, GPU-resident kernel
        records, overheads, MLP features) is stored there and reused by later calls."""
        if not isinstance(operations, (list, tuple)):
            operations = list(operations)
        D = len(dest_devices)
        results = [PredictedOperations(operations, dest) for dest in dest_devices]
        key = ("origins", len(operations))
        by_origin = cache.get(key) if cache is not None else None
        if by_origin is None:
            by_origin = {}
            for i, op in enumerate(operations):
                by_origin.setdefault(op.device.name, []).append(i)
            if cache is not None:
                cache[key] = by_origin
        for origin_name, indices in by_origin.items():
            origin = operations[indices[0]].device
            targets = [d for d in range(D) if dest_devices[d].name != origin_name]
            same = [d for d in range(D) if dest_devices[d].name == origin_name]
            if same:
                ms = np.array([operations[i].run_time_ms for i in indices], np.float64)
                for d in same:
                    results[d].run_times_ms[indices] = ms      # kind 0: the measured operation itself
            if targets:
                self._predict_group(operations, indices, origin, dest_devices, targets, results, cache)
        return results

    # ------------------------------------------------------------------
    def _predict_group(self, operations, indices, origin, dest_devices, targets, results, cache=None):
        dests = [dest_devices[d] for d in targets]
        mode = getattr(self._wave_scaling_strategy, "batch_mode", None)
        key = ("plan", origin.name, mode, len(indices))
        plan = cache.get(key) if cache is not None else None
        if plan is None:
            plan = _GroupPlan(operations, indices, mode)
            if cache is not None:
                cache[key] = plan
        T = len(dests)
        times, totals = self._wave_scale_plan(plan, origin, dests)
        run_ms = (plan.overheads[None, :] + totals) / 1e6                    # [T, runs]
        for t, d in enumerate(targets):
            res = results[d]
            g = len(res._groups)
            res._groups.append(dict(plan=plan, times=times[t], totals=totals[t]))
            if len(plan.wave_idx):
                res._kind[plan.wave_idx] = 1
                res._group[plan.wave_idx] = g
                res._a[plan.wave_idx] = plan.fwd_run
                res._b[plan.wave_idx] = plan.bwd_run
                ms = run_ms[t][plan.fwd_run]
                has_bwd = plan.bwd_run >= 0
                ms = ms + np.where(has_bwd, run_ms[t][np.maximum(plan.bwd_run, 0)], 0.0)
                res.run_times_ms[plan.wave_idx] = ms
            for i in plan.passthrough_idx:
                res._kind[i] = 3
                res.run_times_ms[i] = operations[i].run_time_ms
        for name, idx in plan.mlp_idx.items():
            if not idx:
                continue
            ms = self._special_scale_ops(name, [operations[i] for i in idx], origin, dests, plan)
            idx = np.asarray(idx, np.int64)
            for t, d in enumerate(targets):
                res = results[d]
                res._kind[idx] = 2
                res.run_times_ms[idx] = ms[t]

    def _wave_scale_plan(self, plan, origin, dests):
        """-> (scaled kernel times [T, K], per-pass kernel totals [T, runs]) on the host, float64
        (predictor.py:111-130 of the reference for every pass and destination at once)."""
        T, K, n_runs = len(dests), len(plan.kernels), len(plan.runs)
        if plan.mode is None:
            # a user-supplied strategy: the reference's per-kernel protocol
            times = np.array([[self._wave_scaling_strategy(k, origin, dest, self._kernel_metadata).run_time_ns
                               for k in plan.kernels] for dest in dests], np.float64).reshape(T, K)
            totals = np.zeros((T, n_runs))
            for r in range(n_runs):
                totals[:, r] = times[:, plan.offsets[r]:plan.offsets[r + 1]].sum(axis=1)
            return times, totals
        if K == 0:
            return np.zeros((T, 0)), np.zeros((T, n_runs))
        res = wave_batch.scale_kernels(plan.kernels, origin, dests, self._kernel_metadata, plan.mode,
                                       flat=plan.flat)
        if plan.offsets_dev is None:
            plan.offsets_dev = torch.from_numpy(plan.offsets).cuda()
        # per-pass kernel-time totals on the device: segment sums over the same offsets
        sums = torch.stack([batched.segment_sum(res.scaled_ns[t], plan.offsets_dev) for t in range(T)])
        scaled = res.scaled_ns.cpu().numpy()
        wave_batch.raise_like_reference(scaled)
        return scaled, sums.cpu().numpy()

    def _special_scale_ops(self, name, ops, origin, dests, plan=None):
        """-> [T, n] predicted ms (predictor.py:132-148 and the *_scale methods)."""
        pred = self._predictor(name)
        order = pred.model.features
        cached = plan.mlp_inputs.get(name) if plan is not None else None
        if cached is None:
            cached = (feature_matrix(name, ops, order), np.array([op.run_time_ms for op in ops], np.float32))
            if plan is not None:
                plan.mlp_inputs[name] = cached
        feats, rt_host = cached
        n, T = len(ops), len(dests)
        rows = [pred.device_row(origin.name)] + [pred.device_row(d.name) for d in dests]
        f = torch.from_numpy(np.tile(feats, (T + 1, 1))).cuda()
        r = torch.from_numpy(np.repeat(np.asarray(rows, np.uint8), n)).cuda()
        p = pred.predict_batch(f, r)                      # [(T + 1) n]: origin first
        rt = torch.from_numpy(rt_host).cuda()
        neg = torch.zeros(1, dtype=torch.int32, device="cuda").view(torch.uint32)
        ms = batched.special_scale(rt.repeat(T), p[n:], p[:n].repeat(T), neg).view(T, n).cpu().numpy()
        pred._handle.check_status()
        if int(neg.view(torch.int32).cpu()[0]):
            ph = p.cpu().numpy().astype(np.float64)
            for t in range(T):
                raw = rt_host.astype(np.float64) * ph[(t + 1) * n:(t + 2) * n] / ph[:n]
                for j in np.nonzero(raw < 0)[0]:
                    logger.warning("Operation %s predicted run time %.2f ms", name, raw[j])
        return ms
