"""resimplified wave scaling of a single kernel.

Reference: analyzer/habitat/analysis/wave_scaling/resimplified.py.  Same call signature
(a wave-scaling strategy is any callable (kernel, origin_device, dest_device,
metadata_manager) -> PredictedKernel); the arithmetic runs in the fused device
kernel on a batch of one.  Predictor recognises this function and batches whole
traces instead of calling it per kernel.
"""
from habitat_b200.analysis.kernels import PredictedKernel
from habitat_b200.analysis.wave_scaling import batch


def resimplified_wave_scaling(kernel, origin_device, dest_device, metadata_manager):
    res = batch.scale_kernels([kernel], origin_device, [dest_device], metadata_manager,
                              mode=batch.RESIMPLIFIED)
    scaled = res.scaled_ns.cpu().numpy()
    batch.raise_like_reference(scaled)
    return PredictedKernel(kernel, float(scaled[0, 0]))


resimplified_wave_scaling.batch_mode = batch.RESIMPLIFIED
