"""B200 (sm_100a) grouped-GEMM library with the Python entry points of
DeepLink-org/Triton_Grouped_GEMM.

Sub-packages mirror the reference's module paths:

    triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_TMA.m_grouped_gemm
    triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_masked_TMA.m_grouped_gemm_masked
    triton_grouped_gemm_b200.gemm.BF16.k_grouped_gemm_TMA.k_grouped_gemm
    triton_grouped_gemm_b200.gemm.FP8.*            (per-row/per-expert and block-scaled FP8)
    triton_grouped_gemm_b200.quant.trans_per_block_quant_expand_128x
    triton_grouped_gemm_b200.gemm.layout / .backends

``install_as_reference_modules()`` additionally registers them as top-level ``gemm`` and
``quant`` so code written against the reference (``from gemm.BF16... import ...``) runs
unchanged.  Every operator calls hand-written CUDA through the C ABI in
include/b200gemm.h; there is no Triton, no cuBLAS / CUTLASS / DeepGEMM and no CPU path.
"""

from __future__ import annotations

import importlib
import sys

__version__ = "0.1.0"


def install_as_reference_modules(force: bool = False) -> None:
    """Expose this package's ``gemm`` and ``quant`` as top-level modules of those names."""
    for top in ("gemm", "quant"):
        if top in sys.modules and not force:
            existing = getattr(sys.modules[top], "__file__", "") or ""
            if "triton_grouped_gemm_b200" not in existing:
                raise RuntimeError(f"a different top-level module named {top!r} is already imported")
        mod = importlib.import_module(f"{__name__}.{top}")
        sys.modules[top] = mod
        prefix = f"{__name__}.{top}."
        for name, sub in list(sys.modules.items()):
            if name.startswith(prefix):
                sys.modules[top + "." + name[len(prefix):]] = sub
