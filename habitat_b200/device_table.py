"""Device rows known to the native library.

The C ABI refers to devices by row index in a table uploaded with
hb_set_devices().  This module keeps that table in step with the
DeviceProperties objects Python code passes around: a device is appended (and
the table re-uploaded) the first time it is used.
"""
import ctypes
import os

from habitat_b200 import _native
from habitat_b200.habitat_cuda import DeviceProperties

_DATA_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data")

_rows = []        # spec tuples, index = row
_index = {}       # spec tuple -> row
_uploaded = 0     # number of rows the library has seen
_uploaded_device = None


def load_device_file(path=None):
    """Reads a device table: either this package's row format (columns + devices)
    or the reference's one-mapping-per-device format (data/devices.yml there)."""
    import yaml
    if path is None:
        path = os.path.join(_DATA_DIR, "devices.yml")
    with open(path) as f:
        doc = yaml.safe_load(f)
    out = {}
    if isinstance(doc, dict) and "columns" in doc and "devices" in doc:
        cols = doc["columns"]
        for name, row in doc["devices"].items():
            out[name] = DeviceProperties(name=name, **dict(zip(cols, row)))
    else:
        for name, props in doc.items():
            out[name] = DeviceProperties(name=name, **props)
    return out


def _sync():
    global _uploaded, _uploaded_device
    import torch
    # every GPU of the process gets its own copy inside the library (at its first launch after a
    # change); without a GPU the table still serves the host-side occupancy call
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    if _uploaded == len(_rows) and _uploaded_device == dev:
        return
    lib = _native.load()
    arr = (_native.DeviceSpec * len(_rows))()
    for i, spec in enumerate(_rows):
        arr[i] = _native.DeviceSpec(*spec)
    _native.check(lib.hb_set_devices(arr, len(_rows)))
    _uploaded = len(_rows)
    _uploaded_device = dev


def row_of(device):
    """Row index of a DeviceProperties in the library's table (uploading if new)."""
    spec = device.spec_tuple()
    row = _index.get(spec)
    if row is None:
        if len(_rows) >= _native.HB_MAX_DEVICES:
            raise RuntimeError("device table is full (%d rows)" % _native.HB_MAX_DEVICES)
        row = len(_rows)
        _rows.append(spec)
        _index[spec] = row
    _sync()
    return row


def rows_of(devices):
    rows = [row_of(d) for d in devices]
    _sync()
    return rows


def reset():
    """Forgets every row (tests)."""
    global _uploaded, _uploaded_device
    _rows.clear()
    _index.clear()
    _uploaded = 0
    _uploaded_device = None
