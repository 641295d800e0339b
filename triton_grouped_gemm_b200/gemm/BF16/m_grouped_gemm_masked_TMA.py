"""Masked M-grouped GEMM (drop-in for the reference's gemm/BF16/m_grouped_gemm_masked_TMA.py).

``lhs`` is [G*expected_m, K]; for each group only the first ``masked_m[g]`` rows of its
``expected_m``-row slot are multiplied and written, the rest of ``out`` is left untouched.
Unlike the reference (:185-186) the kernel runs on the caller's current stream, and both
``trans_b`` layouts are implemented (the reference's kernel only handles ``trans_b=True``).
"""

from __future__ import annotations

import torch
from torch import Tensor

from ... import _lib


def m_grouped_gemm_masked(lhs: Tensor, rhs: Tensor, out: torch.Tensor, masked_m: torch.Tensor, expected_m: int,
                          trans_b: bool = True) -> None:
    assert lhs.dim() == 2
    assert rhs.dim() == 3
    M, K = lhs.shape
    assert lhs.stride(-1) == 1, "Please make sure lhs is K-major"
    if trans_b:
        num_groups, N, rhsK = rhs.shape
    else:
        num_groups, rhsK, N = rhs.shape
    assert rhsK == K, "K of lhs should be equal to K of rhs"
    assert (N * rhs.element_size()) % 16 == 0, "TMA required 16-byte alignment"
    assert (K * rhs.element_size()) % 16 == 0, "TMA required 16-byte alignment"
    assert M == num_groups * expected_m, "lhs must hold expected_m rows per group"
    assert out.shape == (M, N), "out should have shape [M, N]"
    code = _lib.dtype_code(lhs.dtype)
    assert rhs.dtype == lhs.dtype and out.dtype == lhs.dtype, "lhs, rhs and out must share one dtype"
    assert lhs.is_contiguous() and rhs.is_contiguous() and out.is_contiguous()
    assert masked_m.numel() == num_groups
    _lib.require_cuda(lhs, rhs, out, masked_m)
    sizes, is64 = _lib.sizes_arg(masked_m)
    lib = _lib.load()
    with torch.cuda.device(lhs.device):
        rc = lib.b200gemm_m_grouped_masked(_lib.ptr(lhs), _lib.ptr(rhs), _lib.ptr(out), _lib.ptr(sizes), is64,
                                           num_groups, int(expected_m), N, K, 1 if trans_b else 0, code, -1,
                                           _lib.stream_ptr(lhs.device))
    _lib.check(rc, "b200gemm_m_grouped_masked")
    return None
