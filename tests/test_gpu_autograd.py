"""Autograd wrapper: forward / dgrad through the M-grouped kernel, wgrad through the K-grouped
kernel, against torch autograd on the per-group fp32 reference."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.gemm.autograd import grouped_gemm

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("trans_b", [True, False])
def test_forward_and_gradients(trans_b):
    sizes = [130, 0, 257, 64]
    m, k, n, g = sum(sizes), 256, 384, len(sizes)
    gen = torch.Generator().manual_seed(3)
    a = (torch.randn(m, k, generator=gen) * 0.5).bfloat16()
    b = (torch.randn(g, n, k, generator=gen) * 0.5).bfloat16()
    if not trans_b:
        b = b.transpose(1, 2).contiguous()
    dc = (torch.randn(m, n, generator=gen) * 0.5).bfloat16()
    # reference: fp32 autograd on the host
    a32 = a.float().requires_grad_(True)
    b32 = b.float().requires_grad_(True)
    outs, row = [], 0
    for i, s in enumerate(sizes):
        w = b32[i].t() if trans_b else b32[i]
        outs.append(a32[row:row + s] @ w)
        row += s
    c_ref = torch.cat(outs)
    c_ref.backward(dc.float())
    # device
    ad = a.to(DEV).requires_grad_(True)
    bd = b.to(DEV).requires_grad_(True)
    c = grouped_gemm(ad, bd, torch.tensor(sizes, device=DEV), trans_b)
    c.backward(dc.to(DEV))
    assert O.rdiff(c.detach().cpu().float(), c_ref.detach()) < 4e-3      # bf16 rounding of the output
    assert O.rdiff(ad.grad.cpu().float(), a32.grad) < 4e-3
    assert O.rdiff(bd.grad.cpu().float(), b32.grad) < 4e-3
    assert torch.all(bd.grad[1] == 0)                                     # empty group -> zero weight gradient
    assert _lib.device_status() == 0


def test_fp8_forward_and_gradients():
    """Block-scaled FP8 forward / input gradient, 16-bit weight gradient, against fp32 autograd on
    the host.  Tolerance: e4m3 with 128-wide scales carries ~2^-4 relative error per element,
    which averages down over the contraction (K = 512, N = 384) to a few per cent of rdiff."""
    from triton_grouped_gemm_b200.gemm.autograd import grouped_gemm_fp8

    sizes = [130, 0, 257, 64]
    m, k, n, g = sum(sizes), 512, 384, len(sizes)
    gen = torch.Generator().manual_seed(4)
    a = torch.randn(m, k, generator=gen).bfloat16()
    b = (torch.randn(g, n, k, generator=gen) * 0.05).bfloat16()
    dc = torch.randn(m, n, generator=gen).bfloat16()
    a32 = a.float().requires_grad_(True)
    b32 = b.float().requires_grad_(True)
    outs, row = [], 0
    for i, s in enumerate(sizes):
        outs.append(a32[row:row + s] @ b32[i].t())
        row += s
    c_ref = torch.cat(outs)
    c_ref.backward(dc.float())
    ad = a.to(DEV).requires_grad_(True)
    bd = b.to(DEV).requires_grad_(True)
    c = grouped_gemm_fp8(ad, bd, torch.tensor(sizes, device=DEV), fp8_wgrad=False)
    c.backward(dc.to(DEV))
    assert c.dtype == torch.bfloat16 and ad.grad.dtype == torch.bfloat16 and bd.grad.dtype == torch.bfloat16
    assert O.rdiff(c.detach().cpu().float(), c_ref.detach()) < 5e-2
    assert O.rdiff(ad.grad.cpu().float(), a32.grad) < 5e-2
    assert O.rdiff(bd.grad.cpu().float(), b32.grad) < 4e-3          # 16-bit weight gradient
    assert torch.all(bd.grad[1] == 0)
    # the all-FP8 recipe (default): the weight gradient comes from e4m3 operands quantised in
    # 128x128 blocks by the transposing quantiser - fp8 noise instead of bf16 noise
    ad8 = a.to(DEV).requires_grad_(True)
    bd8 = b.to(DEV).requires_grad_(True)
    c8 = grouped_gemm_fp8(ad8, bd8, torch.tensor(sizes, device=DEV))
    c8.backward(dc.to(DEV))
    assert torch.equal(c8.detach(), c.detach()) and torch.equal(ad8.grad, ad.grad)
    assert bd8.grad.dtype == torch.bfloat16 and bd8.grad.shape == bd.grad.shape
    assert O.rdiff(bd8.grad.cpu().float(), b32.grad) < 5e-2
    assert not torch.equal(bd8.grad, bd.grad)                        # it really took the FP8 route
    assert torch.all(bd8.grad[1] == 0)
    # and the forward equals the explicit quantise + GEMM path bit for bit
    from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_block_scaled import m_grouped_fp8_block_scaled
    from triton_grouped_gemm_b200.quant.per_block_cast import per_block_cast_to_fp8, per_token_cast_to_fp8

    c2 = m_grouped_fp8_block_scaled(per_token_cast_to_fp8(a.to(DEV)), per_block_cast_to_fp8(b.to(DEV)),
                                    torch.tensor(sizes, device=DEV))
    assert torch.equal(c.detach(), c2)
    assert _lib.device_status() == 0
