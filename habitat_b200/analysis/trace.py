"""An operation trace measured on one device (reference: analyzer/habitat/analysis/trace.py)."""
from habitat_b200.analysis.predictor import Predictor


class Trace:
    # Used when to_device() is called without a predictor.  Created on first
    # use (the reference builds it while the class body is evaluated, which
    # makes importing the package depend on the checkpoint files).
    DefaultPredictor = None

    def __init__(self, device, operations):
        self._device = device
        self._operations = operations
        self._run_time_ms = None
        self._prediction_cache = {}     # flattened kernel records, filled by the first prediction

    @property
    def operations(self):
        return self._operations

    @property
    def device(self):
        return self._device

    @property
    def run_time_ms(self):
        if self._run_time_ms is None:
            total = getattr(self._operations, "total_run_time_ms", None)   # predicted: summed already
            self._run_time_ms = total if total is not None else sum(op.run_time_ms for op in self._operations)
        return self._run_time_ms

    @classmethod
    def _default_predictor(cls):
        if cls.DefaultPredictor is None:
            cls.DefaultPredictor = Predictor()
        return cls.DefaultPredictor

    def to_device(self, dest_device, predictor=None):
        """The predicted trace on `dest_device` (this trace itself if it is the same device)."""
        if dest_device.name == self.device.name:
            return self
        return self.to_devices([dest_device], predictor)[0]

    def to_devices(self, dest_devices, predictor=None):
        """Predicted traces for several destinations from one pass over the kernels."""
        predictor = predictor if predictor is not None else self._default_predictor()
        per_dest = predictor.predict_trace(self._operations, dest_devices, cache=self._prediction_cache)
        return [self if dest.name == self.device.name else Trace(dest, ops)
                for dest, ops in zip(dest_devices, per_dest)]
