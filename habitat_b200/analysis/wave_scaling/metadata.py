"""Per-architecture register counts of known kernels.

Reference: analyzer/habitat/analysis/wave_scaling/metadata.py:7-44, an sqlite
table (name, arch, registers_per_thread) queried once per (kernel, destination).
Here the whole table is read once into a dictionary; `kernel_registers_for`
answers like the reference (largest arch <= the destination's), and
`registers_matrix` resolves a whole batch to the [D, K] array the device path
takes.
"""
import bisect
import logging
import sqlite3

import numpy as np

logger = logging.getLogger(__name__)


def _arch_of(device):
    return int("".join(str(x) for x in device.compute_capability))


class MetadataManager:
    def __init__(self, path_to_lut=None):
        self._by_name = {}
        if path_to_lut is not None:
            connection = sqlite3.connect(path_to_lut)
            try:
                rows = connection.execute(
                    "SELECT name, arch, registers_per_thread FROM kernels").fetchall()
            except sqlite3.OperationalError:
                rows = []   # no such table: an empty look-up table
            finally:
                connection.close()
            for name, arch, regs in rows:
                self._by_name.setdefault(name, []).append((int(arch), int(regs)))
            for entries in self._by_name.values():
                entries.sort()

    def __len__(self):
        return sum(len(v) for v in self._by_name.values())

    def add(self, name, arch, registers_per_thread):
        entries = self._by_name.setdefault(name, [])
        entries.append((int(arch), int(registers_per_thread)))
        entries.sort()

    def _lookup(self, name, arch):
        entries = self._by_name.get(name)
        if not entries:
            return None
        i = bisect.bisect_right(entries, (arch, float("inf")))
        return entries[i - 1] if i else None

    def kernel_registers_for(self, kernel, device):
        arch = _arch_of(device)
        hit = self._lookup(kernel.name, arch)
        if hit is None:
            logger.debug('Missing kernel metadata entry for "%s" on arch %d.', kernel.name, arch)
            return None
        if hit[0] != arch:
            logger.debug('Using substitute entry for "%s" at arch %d instead of %d.',
                         kernel.name, hit[0], arch)
        return hit[1]

    def registers_matrix(self, kernel_names, devices):
        """[D, K] int16, -1 where the table has no entry; None if nothing matched."""
        if not self._by_name:
            return None
        out = np.full((len(devices), len(kernel_names)), -1, dtype=np.int16)
        archs = [_arch_of(d) for d in devices]
        cache = {}
        any_hit = False
        for k, name in enumerate(kernel_names):
            if name not in self._by_name:
                continue
            for d, arch in enumerate(archs):
                key = (name, arch)
                if key not in cache:
                    cache[key] = self._lookup(name, arch)
                hit = cache[key]
                if hit is not None:
                    out[d, k] = hit[1]
                    any_hit = True
        return out if any_hit else None
