"""The reference's optional DeepGEMM entry points (gemm/deep_gemm_ops.py:24-100), served by the
B200 kernels of this package instead of the external ``deep_gemm`` module.

Same names, arguments and layout contract: ``a`` includes each expert's padding rows (every
group padded to ``block_m`` = 128 rows), ``size_per_group`` holds the actual row counts, the
output has the padded shape and its padding rows are not written.  ``grouped_layout`` /
``use_psum_layout`` describe that same layout for DeepGEMM and carry no extra information
here (the kernels derive it from ``size_per_group``); they are accepted and ignored.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from .FP8.m_grouped_gemm_block_scaled import m_grouped_fp8_block_scaled
from .layout import round_up_to_alignment


def _expected_padded_m(size_per_group: torch.Tensor, block_m: int) -> int:
    return int(round_up_to_alignment(size_per_group.to(dtype=torch.int32), block_m).sum().item())


def m_grouped_bf16_nt_contiguous(a: torch.Tensor, b: torch.Tensor, size_per_group: torch.Tensor, *,
                                 out: Optional[torch.Tensor] = None, grouped_layout: Optional[torch.Tensor] = None,
                                 block_m: int = 128, use_psum_layout: bool = False) -> torch.Tensor:
    """BF16 grouped GEMM, NT layout: a [M_padded, K], b [G, N, K] -> [M_padded, N]."""
    del grouped_layout, use_psum_layout
    if a.dim() != 2 or b.dim() != 3:
        raise ValueError("expected a shape [M, K] and b shape [num_groups, N, K]")
    if block_m != 128:
        raise ValueError("the b200 backend pads groups to 128 rows (block_m must be 128)")
    m, k = a.shape
    g, n, bk = b.shape
    if bk != k:
        raise ValueError(f"K mismatch: a has K={k}, b has K={bk}")
    expected_m = _expected_padded_m(size_per_group, block_m)
    if m != expected_m:
        raise ValueError(f"A must include padded expert rows: expected M={expected_m}, got M={m}")
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    _lib.require_cuda(a, b, out, size_per_group)
    assert a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
    sizes, is64 = _lib.sizes_arg(size_per_group)
    with torch.cuda.device(a.device):
        rc = _lib.load().b200gemm_m_grouped_padded(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(sizes), is64, g, m,
                                                   n, k, 1, _lib.dtype_code(a.dtype), -1, _lib.stream_ptr(a.device))
    _lib.check(rc, "b200gemm_m_grouped_padded")
    return out


def m_grouped_fp8_nt_contiguous(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
                                size_per_group: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                                grouped_layout: Optional[torch.Tensor] = None,
                                recipe_a: Optional[Tuple[int, int]] = None,
                                recipe_b: Optional[Tuple[int, int]] = None, block_m: int = 128,
                                use_psum_layout: bool = False) -> torch.Tensor:
    """Block-scaled FP8 grouped GEMM, NT layout.  Scales are fp32: a_scale [M_padded, K/128]
    (recipe (1, 128)), b_scale [G, N/128, K/128] (recipe (128, 128))."""
    del grouped_layout, use_psum_layout
    a_tensor, _ = a
    b_tensor, _ = b
    if a_tensor.dim() != 2 or b_tensor.dim() != 3:
        raise ValueError("expected a[0] shape [M, K] and b[0] shape [num_groups, N, K]")
    if block_m != 128:
        raise ValueError("the b200 backend pads groups to 128 rows (block_m must be 128)")
    if recipe_a not in (None, (1, 128)) or recipe_b not in (None, (128, 128)):
        raise ValueError("the b200 backend implements recipe_a=(1, 128) and recipe_b=(128, 128)")
    m, k = a_tensor.shape
    _, n, bk = b_tensor.shape
    if bk != k:
        raise ValueError(f"K mismatch: a has K={k}, b has K={bk}")
    expected_m = _expected_padded_m(size_per_group, block_m)
    if m != expected_m:
        raise ValueError(f"A must include padded expert rows: expected M={expected_m}, got M={m}")
    return m_grouped_fp8_block_scaled(a, b, size_per_group, out=out, rows_padded=True)
