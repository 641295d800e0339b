"""Transposing 128x128 e4m3 quantiser with per-expert expansion (drop-in for the reference's
quant/trans_per_block_quant_expand_128x.py:135-213).

Output bytes and scales equal the reference's torch implementation
``per_block_trans_quant_expand_torch`` (:253-273) with the one addition its shipped Triton
operator makes: the block scale is clamped to [1e-12, 3e38] (:125).  An all-zero 128x128 block
(zero gradients, a dead column) therefore gives zero bytes and scale 1e-12 instead of the torch
helper's scale 0 and NaN bytes; every block with amax / 448 >= 1e-12 is bit for bit the torch
result."""

from __future__ import annotations

from typing import Tuple

import torch

from .. import _lib


def trans_per_block_quant_expand_128x(input_tensor: torch.Tensor, size_per_group: torch.Tensor,
                                      group_size: int = 128, dtype: torch.dtype = torch.float8_e4m3fn,
                                      ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """input [M, N] -> (fp8 [N, M_EXPAND], scales [N/128, M_EXPAND/128], padded sizes [G]).

    ``M_EXPAND = M + 128*G - M % 128``; each expert's rows are padded to a multiple of 128."""
    M, N = input_tensor.shape
    assert group_size == 128, "only 128x128 blocks are implemented"
    assert N % group_size == 0
    assert dtype == torch.float8_e4m3fn, "only e4m3 output is implemented"
    assert input_tensor.is_contiguous()
    _lib.require_cuda(input_tensor, size_per_group)
    sizes, is64 = _lib.sizes_arg(size_per_group)
    G = sizes.numel()
    m_expand = M + group_size * G - M % group_size
    out = input_tensor.new_empty((N, m_expand), dtype=dtype)
    scales = input_tensor.new_empty((N // group_size, m_expand // group_size), dtype=torch.float32)
    padded = torch.empty(G, device=input_tensor.device, dtype=torch.int64)
    with torch.cuda.device(input_tensor.device):
        rc = _lib.load().b200quant_trans_expand_128x(_lib.ptr(input_tensor), _lib.ptr(sizes), is64, G, _lib.ptr(out),
                                                     _lib.ptr(scales), _lib.ptr(padded), M, N, m_expand,
                                                     _lib.dtype_code(input_tensor.dtype),
                                                     _lib.stream_ptr(input_tensor.device))
    _lib.check(rc, "b200quant_trans_expand_128x")
    return out, scales, padded.to(size_per_group.dtype)


def trans_quant(input_tensor, size_per_group):
    return trans_per_block_quant_expand_128x(input_tensor, size_per_group)
