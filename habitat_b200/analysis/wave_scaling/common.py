"""Occupancy and wave sizes of one kernel on two devices.

Reference: analyzer/habitat/analysis/wave_scaling/common.py:3-20.
"""
from habitat_b200.analysis.wave_scaling import batch


def calculate_wave_info(kernel, origin_device, dest_device, metadata_manager):
    """-> (origin_wave_size, dest_wave_size, origin_occupancy, dest_occupancy)"""
    res = batch.scale_kernels([kernel], origin_device, [dest_device], metadata_manager,
                              mode=batch.RESIMPLIFIED)
    origin_occupancy = int(res.origin_occupancy.cpu()[0])
    dest_occupancy = int(res.dest_occupancy.cpu()[0, 0])
    return (origin_device.num_sms * origin_occupancy, dest_device.num_sms * dest_occupancy,
            origin_occupancy, dest_occupancy)
