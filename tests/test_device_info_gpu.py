"""Device row and peak probe of the local GPU (through the C ABI)."""
import pytest
import torch
import yaml

from habitat_b200 import batched, device_info, device_table, workloads
from habitat_b200.habitat_cuda import KernelInstance

pytestmark = pytest.mark.gpu


def test_device_row_matches_the_driver():
    props = torch.cuda.get_device_properties(0)
    row = device_info.query_device(0, name="local")
    assert row.compute_capability == (props.major, props.minor)
    assert row.num_sms == props.multi_processor_count
    spec = dict(zip(device_info._native.DEVICE_SPEC_FIELDS, row.spec_tuple()))
    assert spec["warp_size"] == props.warp_size
    assert spec["regs_per_multiprocessor"] == props.regs_per_multiprocessor
    assert spec["max_threads_per_multiprocessor"] == props.max_threads_per_multi_processor
    assert spec["shared_mem_per_multiprocessor"] == props.shared_memory_per_multiprocessor
    assert spec["shared_mem_per_block_optin"] == props.shared_memory_per_block_optin
    assert spec["mem_bandwidth_gb"] > 100 and spec["base_clock_mhz"] > 300
    # the row parses back in the reference's YAML form and works as a wave-scaling destination
    doc = yaml.safe_load(device_info.as_yaml(row))
    assert doc["local"]["num_sms"] == props.multi_processor_count
    k = KernelInstance("probe", 1000, 256, 0, 0, 32, 10_000)
    assert 1 <= k.thread_block_occupancy(row) <= 32
    devs = device_table.load_device_file()
    kernels = workloads.make_kernels(1024, seed=3)
    res = batched.wave_scale(batched.KernelBatch.from_numpy(kernels), devs["V100"], [row])
    torch.cuda.synchronize()
    assert res.scaled_ns.shape == (1, 1024)


def test_peak_probe_is_near_the_nominal_peak():
    row = device_info.query_device(0, name="local")
    nominal = dict(zip(device_info._native.DEVICE_SPEC_FIELDS, row.spec_tuple()))["peak_gflops_per_second"]
    measured = device_info.measure_peak_gflops(0, trials=5)
    # an FMA-bound kernel reaches most of lanes x SMs x clock; never more than a little above
    # (the driver reports the maximum clock)
    assert 0.6 * nominal <= measured <= 1.05 * nominal, (measured, nominal)
