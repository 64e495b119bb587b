"""habitat_b200: Habitat's batched prediction path on B200 (sm_100a).

Wave scaling of recorded kernels and inference of the per-operation MLP runtime
predictors, behind the reference analyzer's Python surface.  The arithmetic runs
in hand-written CUDA kernels reached through a C ABI (include/habitat_b200.h);
there is no CPU fallback.
"""
__version__ = "0.1.0"
