"""Analysis data model and predictor (reference: analyzer/habitat/analysis/__init__.py)."""
from habitat_b200.analysis.device import _Device

Device = _Device()

# Operations predicted with an MLP rather than by wave scaling
# (analysis/__init__.py:5-18 of the reference); gru / rnn_* are listed there but
# have no predictor and pass their measured times through.
SPECIAL_OPERATIONS = frozenset({
    "conv2d", "linear", "bmm", "lstm", "gru", "rnn_tanh", "rnn_relu",
})
