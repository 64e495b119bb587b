"""Cross-device prediction of operations and whole traces.

Reference: analyzer/habitat/analysis/predictor.py.  Same constructor, the same
four predictor attributes and the same predict_operation(); what differs is the
inside: instead of one Python call per kernel and two CPU forwards per special
operation, a trace is flattened once and goes through three device launches
(wave scaling, the fused MLP chain per operation kind, the ratio/clamp), for
any number of destination devices at a time (predict_trace).
"""
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
from habitat_b200.utils import ms_to_ns, name_all_arguments, ns_to_ms

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


class Predictor:
    def __init__(self, kernel_metadata_file=None, wave_scaling_strategy=unified_wave_scaling, *,
                 model_paths=None, precision="bf16"):
        if kernel_metadata_file is None:
            default = path_to_data("kernels.sqlite")
            kernel_metadata_file = default if os.path.exists(default) else None
        self._kernel_metadata = MetadataManager(kernel_metadata_file)
        self._wave_scaling_strategy = wave_scaling_strategy
        self._precision = precision
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

        Returns one list of operations per destination, in order; operations
        measured on a device of the same name as the destination are returned
        as they are (analysis/trace.py:40-41 and operation.py:82-85).
        `cache` is a dict the caller keeps with the operations (Trace does): the
        flattened, GPU-resident kernel records are stored there and reused by later
        calls with the same operations."""
        operations = list(operations)
        D = len(dest_devices)
        results = [[None] * len(operations) for _ in range(D)]
        by_origin = {}
        for i, op in enumerate(operations):
            by_origin.setdefault(op.device.name, []).append(i)
        for indices in by_origin.values():
            origin = operations[indices[0]].device
            targets = [d for d in range(D) if dest_devices[d].name != origin.name]
            for d in range(D):
                if d not in targets:
                    for i in indices:
                        results[d][i] = operations[i]
            if targets:
                self._predict_group(operations, indices, origin, dest_devices, targets, results, cache)
        return results

    # ------------------------------------------------------------------
    def _predict_group(self, operations, indices, origin, dest_devices, targets, results, cache=None):
        dests = [dest_devices[d] for d in targets]
        wave_runs = []                     # (op index, is_backward, RunTimeMeasurement)
        mlp_ops = {op: [] for op in _MLP_OPS}
        for i in indices:
            op = operations[i]
            if op.name not in SPECIAL_OPERATIONS:
                wave_runs.append((i, False, op.forward))
                if op.backward is not None:
                    wave_runs.append((i, True, op.backward))
            elif op.name in _MLP_OPS:
                mlp_ops[op.name].append(i)
            else:
                logger.warning("Unhandled special operation: %s", op.name)
                for t, d in enumerate(targets):
                    results[d][i] = PredictedOperation(op, op.forward, op.backward, dests[t])

        wave_out = self._wave_scale_runs(wave_runs, origin, dests, cache) if wave_runs else {}
        for t, d in enumerate(targets):
            fwd, bwd = {}, {}
            for (i, is_bwd, _), pred in zip(wave_runs, wave_out.get(t, [])):
                (bwd if is_bwd else fwd)[i] = pred
            for i, pred in fwd.items():
                results[d][i] = PredictedOperation(operations[i], pred, bwd.get(i), dests[t])

        for name, idx in mlp_ops.items():
            if not idx:
                continue
            ms = self._special_scale_ops(name, [operations[i] for i in idx], origin, dests)
            for t, d in enumerate(targets):
                for j, i in enumerate(idx):
                    results[d][i] = PredictedOperation(
                        operations[i], RunTimePurePrediction(float(ms[t, j]), dests[t]), None, dests[t])

    def _wave_scale_runs(self, wave_runs, origin, dests, cache=None):
        """-> {target index: [RunTimePrediction per run]} (predictor.py:111-130)."""
        kernels, offsets = [], [0]
        for _, _, run in wave_runs:
            kernels.extend(run.kernels)
            offsets.append(len(kernels))
        n_runs, K, T = len(wave_runs), len(kernels), len(dests)
        mode = getattr(self._wave_scaling_strategy, "batch_mode", None)
        if mode is None:
            # a user-supplied strategy: the reference's per-kernel protocol
            out = {}
            for t, dest in enumerate(dests):
                preds = [self._wave_scaling_strategy(k, origin, dest, self._kernel_metadata)
                         for k in kernels]
                out[t] = [self._make_run(run, preds[offsets[r]:offsets[r + 1]], dest, None)
                          for r, (_, _, run) in enumerate(wave_runs)]
            return out
        if K:
            key = ("flat", origin.name, mode)
            flat = cache.get(key) if cache is not None else None
            if flat is None or flat.count != K:
                flat = wave_batch.FlatKernels(kernels, mode)
                if cache is not None:
                    cache[key] = flat
            res = wave_batch.scale_kernels(kernels, origin, dests, self._kernel_metadata, mode, flat=flat)
            # per-run kernel-time totals on the device: [T] segment sums over the same offsets
            off = torch.from_numpy(np.asarray(offsets, np.int64)).cuda()
            sums = torch.stack([batched.segment_sum(res.scaled_ns[t], off) for t in range(T)])
            scaled = res.scaled_ns.cpu().numpy()
            wave_batch.raise_like_reference(res.status.cpu().numpy())
            sums = sums.cpu().numpy()
        else:
            scaled = np.zeros((T, 0), np.float32)
            sums = np.zeros((T, n_runs))
        # per-run overhead (predictor.py:113-116 of the reference) does not depend on the destination
        overheads = []
        for _, _, run in wave_runs:
            overhead_ns = ms_to_ns(run.run_time_ms) - sum(k.run_time_ns for k in run.kernels)
            overheads.append(0 if overhead_ns < 0 else overhead_ns)
        out = {}
        for t, dest in enumerate(dests):
            times = scaled[t].tolist()          # one conversion per destination, not one per kernel
            totals = sums[t].tolist()
            runs = []
            for r in range(n_runs):
                lo, hi = offsets[r], offsets[r + 1]
                preds = [PredictedKernel(kernels[i], times[i]) for i in range(lo, hi)]
                pred = RunTimePrediction(overhead_ns=overheads[r], predicted_kernels=preds, device=dest)
                pred._run_time_ms = ns_to_ms(overheads[r] + totals[r])
                runs.append(pred)
            out[t] = runs
        return out

    @staticmethod
    def _make_run(run, predicted_kernels, dest, kernel_total_ns):
        overhead_ns = ms_to_ns(run.run_time_ms) - sum(k.run_time_ns for k in run.kernels)
        pred = RunTimePrediction(overhead_ns=0 if overhead_ns < 0 else overhead_ns,
                                 predicted_kernels=predicted_kernels, device=dest)
        if kernel_total_ns is not None:
            pred._run_time_ms = ns_to_ms(pred._overhead_ns + kernel_total_ns)
        return pred

    def _special_scale_ops(self, name, ops, origin, dests):
        """-> [T, n] predicted ms (predictor.py:132-148 and the *_scale methods)."""
        pred = self._predictor(name)
        order = pred.model.features
        feats = feature_matrix(name, ops, order)
        n, T = len(ops), len(dests)
        rows = [pred.device_row(origin.name)] + [pred.device_row(d.name) for d in dests]
        f = torch.from_numpy(np.tile(feats, (T + 1, 1))).cuda()
        r = torch.from_numpy(np.repeat(np.asarray(rows, np.uint8), n)).cuda()
        p = pred.predict_batch(f, r)                      # [(T + 1) n]: origin first
        rt = torch.from_numpy(np.array([op.run_time_ms for op in ops], np.float32)).cuda()
        neg = torch.zeros(1, dtype=torch.int32, device="cuda").view(torch.uint32)
        ms = batched.special_scale(rt.repeat(T), p[n:], p[:n].repeat(T), neg).view(T, n).cpu().numpy()
        pred._handle.check_status()
        if int(neg.view(torch.int32).cpu()[0]):
            ph = p.cpu().numpy().astype(np.float64)
            for t in range(T):
                raw = np.array([op.run_time_ms for op in ops]) * ph[(t + 1) * n:(t + 2) * n] / ph[:n]
                for j in np.nonzero(raw < 0)[0]:
                    logger.warning("Operation %s predicted run time %.2f ms", name, raw[j])
        return ms
