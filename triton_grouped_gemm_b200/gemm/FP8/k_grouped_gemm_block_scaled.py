"""Block-scaled FP8 (e4m3) K-grouped GEMM: the expert weight gradient in FP8.

The reference ships the quantiser whose output layout exists for this product
(quant/trans_per_block_quant_expand_128x.py:135-208: transposed, every expert's tokens padded to
128, one scale per 128x128 block) but no kernel that consumes it; here it is a hand-written
sm_100a kernel.  Both operands are such quantiser outputs:

    x = (x_fp8 [M_DIM, M_EXPAND], x_scale [M_DIM/128, M_EXPAND/128] fp32)
    y = (y_fp8 [N_DIM, M_EXPAND], y_scale [N_DIM/128, M_EXPAND/128] fp32)
    out[g, m, n] = sum_{kb of expert g} (sum_{t in kb} x_fp8[m,t] * y_fp8[n,t]) * x_scale[m//128, kb] * y_scale[n//128, kb]  -> bf16
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from ... import _lib
from ...quant.trans_per_block_quant_expand_128x import trans_per_block_quant_expand_128x

Pair = Tuple[Tensor, Tensor]


def k_grouped_fp8_block_scaled(x: Pair, y: Pair, padded_sizes: Tensor, *, out: Optional[Tensor] = None,
                               num_sms: int = -1, balanced: bool = True) -> Tensor:
    """``padded_sizes`` [G]: each expert's token count rounded up to 128 (the quantiser's third
    output); expert g owns the k-blocks after those of the experts before it.  Returns
    [G, M_DIM, N_DIM] bf16; an expert without tokens gives a zero matrix.  ``balanced`` hands the
    tiles out in order of falling token count (a few hundred bytes of scratch from torch's
    stream-ordered allocator per call); without it they go out in expert order."""
    x8, xs = x
    y8, ys = y
    assert x8.dim() == 2 and y8.dim() == 2 and x8.shape[1] == y8.shape[1], "operands are [dim, M_EXPAND] with the same M_EXPAND"
    assert x8.dtype == torch.float8_e4m3fn and y8.dtype == torch.float8_e4m3fn, "operands must be float8_e4m3fn"
    m_dim, m_expand = x8.shape
    n_dim = y8.shape[0]
    assert m_dim % 128 == 0 and n_dim % 128 == 0 and m_expand % 128 == 0, "dimensions must be multiples of 128"
    assert xs.dtype == torch.float32 and tuple(xs.shape) == (m_dim // 128, m_expand // 128), "x_scale shape"
    assert ys.dtype == torch.float32 and tuple(ys.shape) == (n_dim // 128, m_expand // 128), "y_scale shape"
    assert x8.is_contiguous() and y8.is_contiguous() and xs.is_contiguous() and ys.is_contiguous()
    _lib.require_cuda(x8, xs, y8, ys, padded_sizes)
    g = padded_sizes.numel()
    if out is None:
        out = torch.empty((g, m_dim, n_dim), device=x8.device, dtype=torch.bfloat16)
    assert out.shape == (g, m_dim, n_dim) and out.dtype == torch.bfloat16 and out.is_contiguous()
    sizes, is64 = _lib.sizes_arg(padded_sizes)
    ws, ws_bytes = _lib.k_grouped_workspace(g, x8.device) if balanced else (None, 0)
    with torch.cuda.device(x8.device):
        rc = _lib.load().b200gemm_fp8_k_grouped_block(_lib.ptr(x8), _lib.ptr(xs), _lib.ptr(y8), _lib.ptr(ys), _lib.ptr(out),
                                                      _lib.ptr(sizes), is64, g, m_expand, m_dim, n_dim,
                                                      _lib.ptr(ws) if ws is not None else None, ws_bytes, int(num_sms),
                                                      _lib.stream_ptr(x8.device))
    _lib.check(rc, "b200gemm_fp8_k_grouped_block")
    return out


def fp8_wgrad(a: Tensor, grad_out: Tensor, size_per_group: Tensor) -> Tensor:
    """Expert weight gradient in FP8: ``dW[g] = a[rows of g]^T @ grad_out[rows of g]`` with both
    16-bit operands ([M, K] and [M, N], K and N multiples of 128) first put through the
    transposing 128x128 quantiser.  Returns [G, K, N] bf16."""
    aq, a_s, padded = trans_per_block_quant_expand_128x(a, size_per_group)
    gq, g_s, _ = trans_per_block_quant_expand_128x(grad_out, size_per_group)
    return k_grouped_fp8_block_scaled((aq, a_s), (gq, g_s), padded)
