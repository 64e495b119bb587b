"""Operations of a trace (reference: analyzer/habitat/analysis/operation.py)."""


class Operation:
    """A logical operation of the model: a forward pass and maybe a backward one."""

    def __repr__(self):
        return self.name

    @property
    def run_time_ms(self):
        total = self.forward.run_time_ms
        if self.backward is not None:
            total = total + self.backward.run_time_ms
        return total

    @property
    def ktime_ns(self):
        total = self.forward.ktime_ns
        if self.backward is not None:
            total = total + self.backward.ktime_ns
        return total

    @property
    def arguments(self):
        return None

    @property
    def forward(self):
        raise NotImplementedError

    @property
    def backward(self):
        raise NotImplementedError

    @property
    def name(self):
        raise NotImplementedError

    @property
    def device(self):
        raise NotImplementedError

    def to_device(self, dest_device, predictor):
        raise NotImplementedError


class MeasuredOperation(Operation):
    def __init__(self, name, arguments, forward, backward, device):
        self._name = name
        self._arguments = arguments
        self._forward = forward
        self._backward = backward
        self._device = device

    name = property(lambda self: self._name)
    arguments = property(lambda self: self._arguments)
    forward = property(lambda self: self._forward)
    backward = property(lambda self: self._backward)
    device = property(lambda self: self._device)

    def to_device(self, dest_device, predictor):
        if dest_device.name == self._device.name:
            return self
        return predictor.predict_operation(self, dest_device)


class PredictedOperation(Operation):
    def __init__(self, measured_operation, forward, backward, device):
        self._measured_operation = measured_operation
        self._forward = forward
        self._backward = backward
        self._device = device

    name = property(lambda self: self._measured_operation.name)
    arguments = property(lambda self: self._measured_operation.arguments)
    forward = property(lambda self: self._forward)
    backward = property(lambda self: self._backward)
    device = property(lambda self: self._device)

    def to_device(self, dest_device, predictor):
        raise RuntimeError("Cannot make a prediction using a predicted operation.")
