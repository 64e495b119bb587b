"""`Device.<Name>` look-up of GPU rows (reference: analyzer/habitat/analysis/device.py:5-24)."""


class _Device:
    """Attribute access to the device table, loaded on first use."""

    def __init__(self, path=None):
        self._path = path
        self._devices = None

    def _load(self):
        from habitat_b200 import device_table
        self._devices = device_table.load_device_file(self._path)

    def __getattr__(self, device_name):
        if device_name.startswith("_"):
            raise AttributeError(device_name)
        if self._devices is None:
            self._load()
        try:
            return self._devices[device_name]
        except KeyError:
            raise KeyError(device_name) from None

    def names(self):
        if self._devices is None:
            self._load()
        return list(self._devices)
