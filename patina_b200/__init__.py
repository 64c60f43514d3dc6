"""patina_b200 -- B200 (sm_100a) tcgen05 GEMM behind a C ABI, with a thin torch-tensor host API.

The compute path is the CUDA library in `patina_b200/_lib` (built by `patina_b200.build`);
there is no CPU or PyTorch fallback.
"""
from .lib import GemmConfig, GemmPlan  # noqa: F401
from .gemm import (GemmContext, PatinaGemmError, compute_capability, default_context,  # noqa: F401
                   run_gemm)

__all__ = ["GemmConfig", "GemmPlan", "GemmContext", "PatinaGemmError", "compute_capability",
           "default_context", "run_gemm"]
