"""Differentiable grouped GEMM: forward and input gradient through the M-grouped kernel, weight
gradient through the K-grouped kernel (16-bit, and block-scaled FP8 throughout in ``grouped_gemm_fp8``).

The reference keeps forward (``m_grouped_gemm``) and weight gradient (``k_grouped_gemm``) as
separate operators; its vendored baseline wraps the cuBLAS loop in an autograd function
(grouped_gemm/grouped_gemm/ops.py:12-42).  This is the same wrapper over the B200 kernels:

    trans_b=False, B [G, K, N]:  C = A B_g      dA = dC B_g^T (M-grouped, trans_b=True)
                                 dB_g = A_g^T dC_g                (K-grouped) -> [G, K, N]
    trans_b=True,  B [G, N, K]:  C = A B_g^T    dA = dC B_g   (M-grouped, trans_b=False)
                                 dB_g = dC_g^T A_g                (K-grouped) -> [G, N, K]
"""

from __future__ import annotations

import torch

from .BF16.k_grouped_gemm_TMA import k_grouped_gemm
from .BF16.m_grouped_gemm_TMA import _m_grouped_gemm_launch


class _GroupedGemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, size_per_group, trans_b):
        n = b.shape[1] if trans_b else b.shape[2]
        c = a.new_empty(a.shape[0], n)
        _m_grouped_gemm_launch(a.contiguous(), b.contiguous(), c, size_per_group, trans_b)
        ctx.save_for_backward(a, b, size_per_group)
        ctx.trans_b = trans_b
        return c

    @staticmethod
    def backward(ctx, grad):
        a, b, size_per_group = ctx.saved_tensors
        grad = grad.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da = a.new_empty(a.shape)
            _m_grouped_gemm_launch(grad, b.contiguous(), da, size_per_group, not ctx.trans_b)
        if ctx.needs_input_grad[1]:
            sizes = size_per_group if size_per_group.dtype in (torch.int32, torch.int64) else size_per_group.long()
            if ctx.trans_b:
                db = k_grouped_gemm(grad, a.contiguous(), sizes)   # [G, N, K]
            else:
                db = k_grouped_gemm(a.contiguous(), grad, sizes)   # [G, K, N]
        return da, db, None, None


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, size_per_group: torch.Tensor, trans_b: bool = False):
    """``C[rows of g] = a[rows of g] @ (b[g].T if trans_b else b[g])`` with gradients for a and b.
    Rows of ``a`` beyond ``sum(size_per_group)`` get no output and no gradient (uninitialised)."""
    return _GroupedGemm.apply(a, b, size_per_group, trans_b)


class _GroupedGemmFp8(torch.autograd.Function):
    """FP8 training recipe over the block-scaled kernels: forward and input gradient in e4m3 with
    1x128 activation / 128x128 weight scales (quantised on the fly).  Weight gradient: in FP8 as
    well when ``fp8_wgrad`` is set and K and N are multiples of 128 - both operands go through the
    transposing 128x128 quantiser (quant/trans_per_block_quant_expand_128x.py:135-208 of the
    reference, whose layout exists for this) into the block-scaled K-grouped kernel - otherwise
    in the 16-bit K-grouped kernel.  ``b`` is [G, N, K] (the ``trans_b=True`` layout)."""

    @staticmethod
    def forward(ctx, a, b, size_per_group, fp8_wgrad=True):
        from ..quant.per_block_cast import per_block_cast_to_fp8, per_token_cast_to_fp8
        from .FP8.m_grouped_gemm_block_scaled import m_grouped_fp8_block_scaled

        a = a.contiguous()
        b = b.contiguous()
        c = m_grouped_fp8_block_scaled(per_token_cast_to_fp8(a), per_block_cast_to_fp8(b), size_per_group)
        ctx.save_for_backward(a, b, size_per_group)
        ctx.fp8_wgrad = bool(fp8_wgrad) and a.shape[1] % 128 == 0 and b.shape[1] % 128 == 0 and a.dtype == torch.bfloat16
        return c.to(a.dtype)

    @staticmethod
    def backward(ctx, grad):
        from ..quant.per_block_cast import per_block_cast_to_fp8, per_token_cast_to_fp8
        from .FP8.m_grouped_gemm_block_scaled import m_grouped_fp8_block_scaled

        a, b, size_per_group = ctx.saved_tensors
        grad = grad.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            # dA = dC B_g: contraction over N, so the weights are quantised in their [G, K, N] view
            bt8 = per_block_cast_to_fp8(b.transpose(1, 2).contiguous())
            da = m_grouped_fp8_block_scaled(per_token_cast_to_fp8(grad.to(torch.bfloat16)), bt8, size_per_group).to(a.dtype)
        if ctx.needs_input_grad[1]:
            sizes = size_per_group if size_per_group.dtype in (torch.int32, torch.int64) else size_per_group.long()
            if ctx.fp8_wgrad:
                from .FP8.k_grouped_gemm_block_scaled import fp8_wgrad

                db = fp8_wgrad(grad.to(torch.bfloat16), a, sizes).to(b.dtype)   # [G, N, K] from e4m3 operands
            else:
                db = k_grouped_gemm(grad, a, sizes)   # [G, N, K], 16-bit operands, fp32 accumulation
        return da, db, None, None


def grouped_gemm_fp8(a: torch.Tensor, b: torch.Tensor, size_per_group: torch.Tensor, fp8_wgrad: bool = True):
    """``C[rows of g] = a[rows of g] @ b[g].T`` computed in block-scaled FP8 (K and N multiples of
    128 recommended; K % 16 == 0, N % 8 == 0 required), with an FP8 input gradient and an FP8
    weight gradient (16-bit when ``fp8_wgrad`` is False or K / N are not multiples of 128).
    ``a`` [M, K] and ``b`` [G, N, K] are bf16."""
    return _GroupedGemmFp8.apply(a, b, size_per_group, fp8_wgrad)
