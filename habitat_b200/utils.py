"""Small helpers shared by the analysis package (reference: analyzer/habitat/utils.py:46-63)."""


def ns_to_ms(ns):
    return ns / 1e6


def ms_to_ns(ms):
    return ms * 1e6


def name_all_arguments(all_parameters, args, kwargs):
    """Positional and keyword arguments merged into one dict keyed by the
    callee's declared parameter names (positional values win)."""
    named = dict(kwargs)
    named.update(zip(all_parameters, args))
    return named
