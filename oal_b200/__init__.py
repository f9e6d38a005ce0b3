"""B200-native OAL causal grouped-quadratic attention (forward + backward).

Drop-in for the reference's operator surface; all arithmetic runs in the
hand-written sm_100a CUDA library ``liboal_b200.so`` through a C ABI.
"""

from .grouped_quadratic import oal_attention
from .hd_block_gemm import HDParallelBlockPlan, build_hd_block_gemm_plan
from .hd_block_gemm_autograd import check_pending_status
from .hd_block_gemm_adapters import (
    grouped_causal_attention,
    grouped_coefficient_attention,
    prepare_grouped_hd_block_gemm,
    run_prepared_grouped_hd_block_gemm,
)

__all__ = [
    "oal_attention",
    "grouped_causal_attention",
    "grouped_coefficient_attention",
    "prepare_grouped_hd_block_gemm",
    "run_prepared_grouped_hd_block_gemm",
    "build_hd_block_gemm_plan",
    "HDParallelBlockPlan",
    "check_pending_status",
]
