"""Same operator as ``m_grouped_gemm_TMA`` under the module name of the reference's sm_80
variant (gemm/BF16/m_grouped_gemm.py:220-292).  The reference registers the custom op
``moe::m_grouped_gemm`` in both files; here it is registered once and re-exported."""

from .m_grouped_gemm_TMA import (  # noqa: F401
    _build_m_grouped_metadata,
    _m_grouped_gemm_launch,
    m_grouped_gemm,
    m_grouped_reference,
)
