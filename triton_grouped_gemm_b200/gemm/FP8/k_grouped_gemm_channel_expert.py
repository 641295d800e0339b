"""FP8 K-grouped GEMM with per-(row, group) scales (drop-in for the reference's
gemm/FP8/k_grouped_gemm_channel_expert.py:143-181).

``out[g] = (X[:, ks:ke] . Y[:, ks:ke]^T) * x_scale[m, g] * y_scale[n, g]`` -> bf16 [G, M, N].
``x_fp8`` is [M, K_total] and ``y_fp8`` [N, K_total], both K-major; each group's token count is
a multiple of 128 with zero-padded data; the scale tensors are logical [M, G] / [N, G] whose
memory is group-major (element (m, g) at g*M + m), exactly as the reference's kernel indexes
them (:121-124).
"""

from __future__ import annotations

import torch

from ... import _lib
from .m_grouped_gemm_channel_expert import fp8_code


def _group_major_scale(scale: torch.Tensor, rows: int, groups: int) -> torch.Tensor:
    assert scale.dtype == torch.float32
    assert scale.numel() == rows * groups, "scale must hold rows * num_groups values"
    if scale.dim() == 2 and tuple(scale.shape) == (rows, groups) and groups > 1 and rows > 1:
        assert scale.stride() == (1, rows), "scale [rows, groups] must be group-major in memory (stride (1, rows))"
        return scale
    assert scale.is_contiguous() or scale.t().is_contiguous()
    return scale


def matmul(x_fp8: torch.Tensor, x_scale: torch.Tensor, y_fp8: torch.Tensor, y_scale: torch.Tensor,
           tokens_per_expert: torch.Tensor, M: int, N: int, K: int, num_groups: int, dtype_a: int = 1,
           dtype_b: int = 1) -> torch.Tensor:
    """``dtype_a`` / ``dtype_b``: 1 = e4m3, anything else = e5m2 (reference convention)."""
    assert x_fp8.shape == (M, K) and y_fp8.shape == (N, K), "x_fp8 is [M, K_total], y_fp8 is [N, K_total]"
    assert x_fp8.is_contiguous() and y_fp8.is_contiguous()
    assert tokens_per_expert.numel() == num_groups
    _lib.require_cuda(x_fp8, x_scale, y_fp8, y_scale, tokens_per_expert)
    assert fp8_code(x_fp8.dtype) == (0 if dtype_a == 1 else 1), "dtype_a does not match x_fp8.dtype"
    assert fp8_code(y_fp8.dtype) == (0 if dtype_b == 1 else 1), "dtype_b does not match y_fp8.dtype"
    xs = _group_major_scale(x_scale, M, num_groups)
    ys = _group_major_scale(y_scale, N, num_groups)
    sizes, is64 = _lib.sizes_arg(tokens_per_expert)
    out = torch.empty((num_groups, M, N), dtype=torch.bfloat16, device=x_fp8.device)
    with torch.cuda.device(x_fp8.device):
        ws, ws_bytes = _lib.k_grouped_workspace(num_groups, x_fp8.device)
        rc = _lib.load().b200gemm_fp8_k_grouped_rowcol(
            _lib.ptr(x_fp8), _lib.ptr(xs), _lib.ptr(y_fp8), _lib.ptr(ys), _lib.ptr(out), _lib.ptr(sizes), is64,
            num_groups, K, M, N, fp8_code(x_fp8.dtype), fp8_code(y_fp8.dtype),
            _lib.ptr(ws) if ws is not None else None, ws_bytes, -1, _lib.stream_ptr(x_fp8.device))
    _lib.check(rc, "b200gemm_fp8_k_grouped_rowcol")
    return out
