"""Same operator as ``k_grouped_gemm_TMA`` under the module name of the reference's sm_80
variant (gemm/BF16/k_grouped_gemm.py:142-216)."""

from typing import Optional

from torch import Tensor

from .k_grouped_gemm_TMA import gmm_dw_reference  # noqa: F401
from .k_grouped_gemm_TMA import k_grouped_gemm as _k_grouped_gemm


def k_grouped_gemm(A: Tensor, B: Tensor, size_per_group: Tensor, group_start: Optional[Tensor] = None,
                   group_end: Optional[Tensor] = None) -> Tensor:
    return _k_grouped_gemm(A, B, size_per_group, group_start, group_end)
