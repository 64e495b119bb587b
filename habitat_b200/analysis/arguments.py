"""Recorded call arguments of an operation (reference: analyzer/habitat/analysis/arguments.py)."""


def _shape_of(value):
    """Tensors are kept as their sizes only; containers are walked; scalars pass."""
    if isinstance(value, tuple):
        return tuple(_shape_of(v) for v in value)
    if isinstance(value, list):
        return [_shape_of(v) for v in value]
    size = getattr(value, "size", None)
    if callable(size) and hasattr(value, "dtype") and hasattr(value, "dim"):
        return value.size()
    return value


class Arguments:
    def __init__(self, args, kwargs):
        self.args = args
        self.kwargs = kwargs
        self.special = {}

    @classmethod
    def from_raw_arguments(cls, args, kwargs):
        return cls(tuple(_shape_of(a) for a in args), {k: _shape_of(v) for k, v in kwargs.items()})
