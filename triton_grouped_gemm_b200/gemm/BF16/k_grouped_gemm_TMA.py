"""BF16 / FP16 K-grouped GEMM, the expert weight gradient (drop-in for the reference's
gemm/BF16/k_grouped_gemm_TMA.py:183-294).

``C[g] = A[gs:ge].T @ B[gs:ge]`` for A [K_TOTAL, M_DIM], B [K_TOTAL, N_DIM] ->
C [G, M_DIM, N_DIM].  No group-level padding; an empty group gives zeros.  Unlike the
reference there is no M_DIM % BLOCK_M / N_DIM % BLOCK_N restriction (only the 16-byte row
alignment TMA needs).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from ... import _lib


def _dtype_code(dtype: torch.dtype) -> int:
    return _lib.dtype_code(dtype)


def _check_k_grouped_gemm_inputs(A: Tensor, B: Tensor, size_per_group: Tensor,
                                 trans_b: bool = False) -> Tuple[int, int, int, int]:
    """Same checks and messages as the reference (:183-214)."""
    assert not trans_b, ("trans_b=True path has been removed; pass B as contiguous [K_TOTAL, N_DIM] "
                         "and trans_b=False")
    assert A.is_cuda and B.is_cuda and size_per_group.is_cuda, "A, B, and size_per_group must be CUDA tensors"
    assert A.dim() == 2, "A must be 2D"
    assert B.dim() == 2, "B must be 2D"
    assert A.is_contiguous(), "A must be contiguous [K_TOTAL, M_DIM]"
    assert B.is_contiguous(), "B must be contiguous [K_TOTAL, N_DIM]"
    assert size_per_group.dim() == 1, "size_per_group must be 1D"
    assert size_per_group.dtype in (torch.int32, torch.int64), "size_per_group must be int32 or int64"
    K_TOTAL, M_DIM = A.shape
    K_B, N_DIM = B.shape
    assert K_TOTAL == K_B, f"A K_TOTAL={K_TOTAL} must equal B K_TOTAL={K_B}"
    _dtype_code(A.dtype)
    _dtype_code(B.dtype)
    assert A.dtype == B.dtype, f"A dtype {A.dtype} and B dtype {B.dtype} should match"
    assert A.data_ptr() % 16 == 0, "A base pointer must be 16-byte aligned for TMA path"
    assert B.data_ptr() % 16 == 0, "B base pointer must be 16-byte aligned for TMA path"
    assert (M_DIM * A.element_size()) % 16 == 0, "A row stride must be 16-byte aligned for TMA path"
    assert (N_DIM * B.element_size()) % 16 == 0, "B row stride must be 16-byte aligned for TMA path"
    return K_TOTAL, M_DIM, N_DIM, int(size_per_group.numel())


def k_grouped_gemm(A: Tensor, B: Tensor, size_per_group: Tensor, group_start: Optional[Tensor] = None,
                   group_end: Optional[Tensor] = None, trans_b: bool = False, numSM: int = -1,
                   use_fixed_sm90_config: bool = True) -> Tensor:
    del use_fixed_sm90_config
    K_TOTAL, M_DIM, N_DIM, num_groups = _check_k_grouped_gemm_inputs(A, B, size_per_group, trans_b)
    C = A.new_empty(num_groups, M_DIM, N_DIM)
    gs = ge = None
    if group_start is not None and group_end is not None:
        gs = group_start.to(torch.int32).contiguous()
        ge = group_end.to(torch.int32).contiguous()
    sizes, is64 = _lib.sizes_arg(size_per_group)
    with torch.cuda.device(A.device):
        ws, ws_bytes = _lib.k_grouped_workspace(num_groups, A.device)
        rc = _lib.load().b200gemm_k_grouped(
            _lib.ptr(A), _lib.ptr(B), _lib.ptr(C), _lib.ptr(sizes), is64,
            _lib.ptr(gs) if gs is not None else None, _lib.ptr(ge) if ge is not None else None,
            num_groups, K_TOTAL, M_DIM, N_DIM, _dtype_code(A.dtype), _lib.ptr(ws) if ws is not None else None,
            ws_bytes, int(numSM), _lib.stream_ptr(A.device))
    _lib.check(rc, "b200gemm_k_grouped")
    return C


def gmm_dw_reference(a: Tensor, b: Tensor, batch_sizes_cpu: Tensor) -> Tensor:
    """Per-group torch product, the correctness baseline (reference :402-416)."""
    out = a.new_zeros(batch_sizes_cpu.numel(), a.shape[1], b.shape[1])
    row = 0
    for g, rows in enumerate(batch_sizes_cpu.tolist()):
        out[g] = a[row:row + rows].T @ b[row:row + rows]
        row += rows
    return out.contiguous()
