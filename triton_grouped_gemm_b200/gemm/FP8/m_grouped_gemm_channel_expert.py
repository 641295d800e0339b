"""FP8 M-grouped GEMM with per-row activation scales and per-expert-per-channel weight scales
(drop-in for the reference's gemm/FP8/m_grouped_gemm_channel_expert.py:139-198).

``C[m, n] = (A_fp8[m] . B_fp8[g, n]) * A_scale[m] * B_scale[g*N + n]``, fp32 accumulation over
the whole K, one rounding to ``dtype_out``.  e4m3 and e5m2 operands in any combination.
The torch cast helpers the reference keeps under ``__main__`` (:217-261) are importable here.
"""

from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from ... import _lib

_FP8_CODE = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}


def fp8_code(dtype: torch.dtype) -> int:
    assert dtype in _FP8_CODE, f"data type {dtype} is not an fp8 type this backend supports"
    return _FP8_CODE[dtype]


@torch.library.custom_op("myfp8::gmm_fp8_act_per_channel_w_per_expert", mutates_args=())
def gmm_fp8_act_per_channel_w_per_expert(A: Tensor, A_scale: Tensor, B: Tensor, B_scale: torch.Tensor,
                                         size_per_group: torch.Tensor,
                                         dtype_out: torch.dtype = torch.float16) -> Tensor:
    assert A.dim() == 2
    assert B.dim() == 3
    M, K = A.shape
    num_groups, N, BK = B.shape
    assert BK == K
    assert B.stride(-1) == 1, "Please make sure B is K-major"
    assert A.stride(-1) == 1, "Please make sure A is K-major"
    assert A.is_contiguous() and B.is_contiguous()
    assert A_scale.numel() == M and B_scale.numel() == num_groups * N, "A_scale is [M], B_scale is [G*N]"
    assert A_scale.dtype == torch.float32 and B_scale.dtype == torch.float32
    assert dtype_out in (torch.float16, torch.bfloat16)
    assert size_per_group.numel() == num_groups
    _lib.require_cuda(A, A_scale, B, B_scale, size_per_group)
    a_s = A_scale.reshape(-1).contiguous()
    b_s = B_scale.reshape(-1).contiguous()
    sizes, is64 = _lib.sizes_arg(size_per_group)
    C = A.new_empty(M, N, dtype=dtype_out)
    with torch.cuda.device(A.device):
        rc = _lib.load().b200gemm_fp8_m_grouped_rowcol(
            _lib.ptr(A), _lib.ptr(a_s), _lib.ptr(B), _lib.ptr(b_s), _lib.ptr(C), _lib.ptr(sizes), is64, num_groups, M,
            N, K, fp8_code(A.dtype), fp8_code(B.dtype), _lib.dtype_code(dtype_out), -1, _lib.stream_ptr(A.device))
    _lib.check(rc, "b200gemm_fp8_m_grouped_rowcol")
    return C


@gmm_fp8_act_per_channel_w_per_expert.register_fake
def _(A, A_scale, B, B_scale, size_per_group, dtype_out=torch.float16):
    return A.new_empty(A.shape[0], B.shape[1], dtype=dtype_out)


def ceil_div(x: int, y: int) -> int:
    return (x + y - 1) // y


def per_channel_cast_to_fp8(x: Tensor, dtype=torch.float8_e4m3fn) -> Tuple[Tensor, Tensor]:
    """One scale per row (torch; test-data helper of the reference, :224-234)."""
    assert x.dim() == 2 and x.size(1) % 128 == 0
    m, n = x.shape
    amax = x.abs().float().amax(dim=1, keepdim=True).clamp(1e-4)
    fmax = torch.finfo(dtype).max
    return (x * (fmax / amax)).to(dtype), (amax / fmax).view(m, 1)


def per_expert_cast_to_fp8(x: Tensor, dtype=torch.float8_e4m3fn) -> Tuple[Tensor, Tensor]:
    """One scale per expert (torch; test-data helper of the reference, :247-261)."""
    assert x.dim() == 3
    g = x.shape[0]
    amax = x.abs().float().amax(dim=(1, 2), keepdim=True).clamp(1e-4)
    fmax = torch.finfo(dtype).max
    return (x * (fmax / amax)).to(dtype).contiguous(), (amax / fmax).view(g, 1)
