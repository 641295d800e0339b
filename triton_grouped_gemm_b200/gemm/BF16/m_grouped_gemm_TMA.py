"""BF16 / FP16 M-grouped GEMM (drop-in for the reference's gemm/BF16/m_grouped_gemm_TMA.py).

``C[rows of g] = A[rows of g] @ B_g`` with fp32 accumulation.  The reference builds tile
metadata with ~10 small torch ops and a host sync, then launches a Triton kernel
(gemm/BF16/m_grouped_gemm_TMA.py:297-432); here one persistent sm_100a kernel walks
``size_per_group`` on the device, so a call is a single launch with no synchronisation.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ... import _lib
from ..layout import device_group_metadata

BLOCK_M = 128


def _build_m_grouped_metadata(size_per_group: Tensor, block_m: int = 128):
    """Same tuple as the reference (:297-326).  The B200 kernel does not need it; it is kept
    because benchmark code builds it once and passes it as ``metadata=``."""
    return device_group_metadata(size_per_group, block_m)


def _m_grouped_gemm_launch(A: Tensor, B: Tensor, C: Tensor, size_per_group: Tensor, trans_b: bool = False,
                           numSM: int = -1, metadata=None, use_fixed_sm90_config: bool = True) -> Tensor:
    """Checks mirror the reference's asserts (:338-374); ``metadata`` and
    ``use_fixed_sm90_config`` are accepted and ignored."""
    del metadata, use_fixed_sm90_config
    assert A.dim() == 2
    assert B.dim() == 3
    assert C.dim() == 2
    M, K = A.shape
    if trans_b:
        num_groups, N, BK = B.shape
    else:
        num_groups, BK, N = B.shape
    assert BK == K, "K of A should be equal to K of B"
    assert C.shape == (M, N), "C should have shape [M, N]"
    assert A.stride(-1) == 1, "Please make sure A is K-major"
    code = _lib.dtype_code(A.dtype)
    assert B.dtype == A.dtype and C.dtype == A.dtype, "A, B and C must share one dtype"
    assert (N * B.element_size()) % 16 == 0, "TMA required 16-byte alignment"
    assert (K * B.element_size()) % 16 == 0, "TMA required 16-byte alignment"
    assert A.is_contiguous() and B.is_contiguous() and C.is_contiguous(), "A, B and C must be contiguous"
    assert size_per_group.numel() == num_groups, "size_per_group must have one entry per group"
    _lib.require_cuda(A, B, C, size_per_group)
    sizes, is64 = _lib.sizes_arg(size_per_group)
    lib = _lib.load()
    with torch.cuda.device(A.device):
        rc = lib.b200gemm_m_grouped(_lib.ptr(A), _lib.ptr(B), _lib.ptr(C), _lib.ptr(sizes), is64, num_groups, M, N, K,
                                    1 if trans_b else 0, code, int(numSM), _lib.stream_ptr(A.device))
    _lib.check(rc, "b200gemm_m_grouped")
    return C


@torch.library.custom_op("moe::m_grouped_gemm", mutates_args=())
def m_grouped_gemm(A: Tensor, B: Tensor, size_per_group: torch.Tensor, trans_b: bool = False,
                   numSM: int = -1) -> Tensor:
    M, K = A.shape
    N = B.shape[1] if trans_b else B.shape[2]
    C = A.new_empty(M, N)
    return _m_grouped_gemm_launch(A, B, C, size_per_group, trans_b, numSM)


@m_grouped_gemm.register_fake
def _(A: Tensor, B: Tensor, size_per_group: torch.Tensor, trans_b: bool = False, numSM: int = -1) -> Tensor:
    M, K = A.shape
    N = B.shape[1] if trans_b else B.shape[2]
    return A.new_empty(M, N)


def m_grouped_reference(a: Tensor, b: Tensor, batch_sizes_cpu: Tensor, trans_b: bool) -> Tensor:
    """Per-group torch product, the correctness baseline (reference :573-581)."""
    pieces, row = [], 0
    for g, rows in enumerate(batch_sizes_cpu.tolist()):
        w = b[g].t() if trans_b else b[g]
        pieces.append(a[row:row + rows] @ w)
        row += rows
    return torch.cat(pieces).contiguous()
