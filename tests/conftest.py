import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def device_file():
    from habitat_b200 import device_table
    return device_table.load_device_file()


@pytest.fixture(scope="session")
def bench_devices(device_file):
    from habitat_b200 import workloads
    return [device_file[n] for n in workloads.BENCH_DEVICES]
