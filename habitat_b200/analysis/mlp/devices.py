"""Device feature rows of the MLP predictors.

Reference: analyzer/habitat/analysis/mlp/devices.py:5-21, which re-reads
devices.csv with pandas on every predict() call.  Here the table is parsed once
and cached; look-ups are by device name, as in the reference.
"""
import csv
import os

from habitat_b200.data import path_to_data

_cache = {}


def _table(path=None):
    path = path or path_to_data("mlp_devices.csv")
    key = os.path.abspath(path)
    if key not in _cache:
        with open(key, newline="") as f:
            rows = list(csv.DictReader(f))
        _cache[key] = {r["device"]: r for r in rows}
    return _cache[key]


def get_device_features(device_name, device_params, path=None):
    """Values of `device_params` for one device, in that order."""
    table = _table(path)
    if device_name not in table:
        raise IndexError("device %r is not in the MLP device table" % (device_name,))
    return [float(table[device_name][p]) for p in device_params]


def get_all_devices(device_params=None, path=None):
    table = _table(path)
    out = {}
    for name, row in table.items():
        keys = device_params if isinstance(device_params, list) else [k for k in row if k != "device"]
        out[name] = [float(row[k]) if row[k] != "" else float("nan") for k in keys]
    return out


def register_device(device_name, features, device_params=("mem", "mem_bw", "num_sm", "single"),
                    path=None):
    """Adds (or replaces) a row at run time, e.g. for a GPU the table lacks."""
    row = {"device": device_name}
    row.update({p: str(v) for p, v in zip(device_params, features)})
    _table(path)[device_name] = row
