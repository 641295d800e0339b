"""1x128 and 128x128 e4m3 quantisers on the GPU.

The reference has these only as torch helpers inside ``__main__`` blocks
(gemm/FP8/m_grouped_gemm_channel_expert.py:217-245); the CUDA kernels reproduce their bytes
and scales exactly."""

from __future__ import annotations

from typing import Tuple

import torch

from .. import _lib


def per_token_cast_to_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [m, k] bf16/fp16, k % 128 == 0 -> (e4m3 [m, k], fp32 scales [m, k/128])."""
    assert x.dim() == 2 and x.size(1) % 128 == 0
    assert x.is_contiguous()
    _lib.require_cuda(x)
    m, k = x.shape
    q = torch.empty((m, k), device=x.device, dtype=torch.float8_e4m3fn)
    s = torch.empty((m, k // 128), device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        rc = _lib.load().b200quant_act_1x128(_lib.ptr(x), _lib.ptr(q), _lib.ptr(s), m, k, _lib.dtype_code(x.dtype),
                                             _lib.stream_ptr(x.device))
    _lib.check(rc, "b200quant_act_1x128")
    return q, s


def per_block_cast_to_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [m, n] (or [batch, m, n]) -> (e4m3 same shape, fp32 scales [..., ceil(m/128), ceil(n/128)])."""
    assert x.dim() in (2, 3)
    assert x.is_contiguous()
    _lib.require_cuda(x)
    batch = 1 if x.dim() == 2 else x.shape[0]
    m, n = x.shape[-2:]
    q = torch.empty(x.shape, device=x.device, dtype=torch.float8_e4m3fn)
    sshape = ((m + 127) // 128, (n + 127) // 128)
    if x.dim() == 3:
        sshape = (batch,) + sshape
    s = torch.empty(sshape, device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        rc = _lib.load().b200quant_w_128x128(_lib.ptr(x), _lib.ptr(q), _lib.ptr(s), batch, m, n,
                                             _lib.dtype_code(x.dtype), _lib.stream_ptr(x.device))
    _lib.check(rc, "b200quant_w_128x128")
    return q, s


def swiglu_per_token_cast_to_fp8(h: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """h [rows, 2*inter] bf16 holding gate | up -> (e4m3 [rows, inter], scales [rows, inter/128]) of
    bf16(silu(gate) * up), in one pass (inter % 128 == 0)."""
    assert h.dim() == 2 and h.dtype == torch.bfloat16 and h.is_contiguous()
    rows, two_i = h.shape
    inter = two_i // 2
    assert two_i == 2 * inter and inter % 128 == 0
    _lib.require_cuda(h)
    q = torch.empty((rows, inter), device=h.device, dtype=torch.float8_e4m3fn)
    s = torch.empty((rows, inter // 128), device=h.device, dtype=torch.float32)
    with torch.cuda.device(h.device):
        rc = _lib.load().b200quant_swiglu_act_1x128(_lib.ptr(h), _lib.ptr(q), _lib.ptr(s), rows, inter,
                                                    _lib.stream_ptr(h.device))
    _lib.check(rc, "b200quant_swiglu_act_1x128")
    return q, s
