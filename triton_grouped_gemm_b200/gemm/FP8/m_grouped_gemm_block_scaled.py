"""Block-scaled FP8 (e4m3) M-grouped GEMMs: 1x128 activation scales x 128x128 weight scales.

The reference reaches this operation only through an external package
(gemm/deep_gemm_ops.py:60-100); here it is a hand-written sm_100a kernel.  Inputs are what
``per_token_cast_to_fp8`` / ``per_block_cast_to_fp8`` produce:

    a = (a_fp8 [M, K], a_scale [M, ceil(K/128)] fp32)
    b = (b_fp8 [G, N, K], b_scale [G, ceil(N/128), ceil(K/128)] fp32)
    C[m, n] = sum_kb (sum_{k in kb} a_fp8[m,k] * b_fp8[g,n,k]) * a_scale[m,kb] * b_scale[g,n//128,kb]  -> bf16
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from ... import _lib

Pair = Tuple[Tensor, Tensor]


def _check_pairs(a: Pair, b: Pair):
    a8, a_s = a
    b8, b_s = b
    assert a8.dim() == 2 and b8.dim() == 3, "expected a[0] shape [M, K] and b[0] shape [num_groups, N, K]"
    m, k = a8.shape
    g, n, bk = b8.shape
    assert bk == k, f"K mismatch: a has K={k}, b has K={bk}"
    assert a8.dtype == torch.float8_e4m3fn and b8.dtype == torch.float8_e4m3fn, "operands must be float8_e4m3fn"
    kb, nb = (k + 127) // 128, (n + 127) // 128
    assert a_s.dtype == torch.float32 and tuple(a_s.shape) == (m, kb), f"a_scale must be fp32 [{m}, {kb}]"
    assert b_s.dtype == torch.float32 and tuple(b_s.shape) == (g, nb, kb), f"b_scale must be fp32 [{g}, {nb}, {kb}]"
    assert a8.is_contiguous() and b8.is_contiguous() and a_s.is_contiguous() and b_s.is_contiguous()
    assert k % 16 == 0, "TMA required 16-byte alignment"
    assert n % 8 == 0, "N must be a multiple of 8"
    _lib.require_cuda(a8, a_s, b8, b_s)
    return a8, a_s, b8, b_s, m, n, k, g


def m_grouped_fp8_block_scaled(a: Pair, b: Pair, size_per_group: Tensor, *, out: Optional[Tensor] = None,
                               rows_padded: bool = False, num_sms: int = -1,
                               group_to_b: Optional[Tensor] = None) -> Tensor:
    """``rows_padded=False``: rows of ``a`` are compact (sum(size_per_group) rows used).
    ``rows_padded=True``: each group's rows are padded to a multiple of 128 (DeepGEMM's
    contiguous layout); padding rows of ``out`` are not written.  ``num_sms`` > 0 limits the
    persistent grid (e.g. to leave SMs to a collective running beside the GEMM).
    ``group_to_b`` (int32, one entry per row group): row group i uses ``b[group_to_b[i]]``; the
    number of row groups is then ``size_per_group.numel()``, independent of ``b.shape[0]``."""
    a8, a_s, b8, b_s, m, n, k, g = _check_pairs(a, b)
    _lib.require_cuda(size_per_group)
    if group_to_b is not None:
        assert not rows_padded, "group_to_b works on compact rows"
        assert group_to_b.dtype == torch.int32 and group_to_b.is_contiguous()
        assert group_to_b.numel() == size_per_group.numel()
        _lib.require_cuda(group_to_b)
        if out is None:
            out = torch.empty((m, n), device=a8.device, dtype=torch.bfloat16)
        assert out.shape == (m, n) and out.dtype == torch.bfloat16 and out.is_contiguous()
        sizes, is64 = _lib.sizes_arg(size_per_group)
        with torch.cuda.device(a8.device):
            rc = _lib.load().b200gemm_fp8_m_grouped_block_mapped(
                _lib.ptr(a8), _lib.ptr(a_s), _lib.ptr(b8), _lib.ptr(b_s), _lib.ptr(out), _lib.ptr(sizes), is64,
                size_per_group.numel(), _lib.ptr(group_to_b), g, m, n, k, int(num_sms), _lib.stream_ptr(a8.device))
        _lib.check(rc, "b200gemm_fp8_m_grouped_block_mapped")
        return out
    assert size_per_group.numel() == g
    if out is None:
        out = torch.empty((m, n), device=a8.device, dtype=torch.bfloat16)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16 and out.is_contiguous()
    sizes, is64 = _lib.sizes_arg(size_per_group)
    with torch.cuda.device(a8.device):
        rc = _lib.load().b200gemm_fp8_m_grouped_block(
            _lib.ptr(a8), _lib.ptr(a_s), _lib.ptr(b8), _lib.ptr(b_s), _lib.ptr(out), _lib.ptr(sizes), is64, g, m, n, k,
            1 if rows_padded else 0, int(num_sms), _lib.stream_ptr(a8.device))
    _lib.check(rc, "b200gemm_fp8_m_grouped_block")
    return out


def m_grouped_fp8_block_scaled_masked(a: Pair, b: Pair, out: Tensor, masked_m: Tensor, expected_m: int) -> None:
    """Masked (decode) layout: ``a[0]`` is [G*expected_m, K]; rows [g*expected_m,
    g*expected_m + masked_m[g]) of ``out`` are written, the rest is left untouched."""
    a8, a_s, b8, b_s, m, n, k, g = _check_pairs(a, b)
    assert m == g * expected_m, "a must hold expected_m rows per group"
    assert out.shape == (m, n) and out.dtype == torch.bfloat16 and out.is_contiguous()
    assert masked_m.numel() == g
    _lib.require_cuda(out, masked_m)
    sizes, is64 = _lib.sizes_arg(masked_m)
    with torch.cuda.device(a8.device):
        rc = _lib.load().b200gemm_fp8_m_grouped_masked_block(
            _lib.ptr(a8), _lib.ptr(a_s), _lib.ptr(b8), _lib.ptr(b_s), _lib.ptr(out), _lib.ptr(sizes), is64, g,
            int(expected_m), n, k, -1, _lib.stream_ptr(a8.device))
    _lib.check(rc, "b200gemm_fp8_m_grouped_masked_block")
    return None


def interleave_gate_up(w13: Tensor) -> Tensor:
    """[..., 2*I, H] with gate rows then up rows -> the same rows interleaved in 128-row blocks
    (gate block 0, up block 0, gate block 1, ...), the weight layout of the SwiGLU-epilogue GEMM.
    128x128 quantisation commutes with this permutation (it moves whole scale blocks)."""
    two_i, h = w13.shape[-2:]
    assert two_i % 256 == 0, "the intermediate size must be a multiple of 128"
    lead = w13.shape[:-2]
    return w13.reshape(*lead, 2, two_i // 256, 128, h).transpose(-4, -3).reshape(*lead, two_i, h).contiguous()


def m_grouped_fp8_block_scaled_swiglu(a: Pair, b_interleaved: Pair, size_per_group: Tensor, *, masked_stride: int = 0,
                                      group_to_b: Optional[Tensor] = None, num_sms: int = -1) -> Pair:
    """Gate+up GEMM with SwiGLU and the 1x128 quantiser in its epilogue.  ``b_interleaved`` is the
    quantised ``interleave_gate_up(w13)``.  Returns (act e4m3 [M, I], scales fp32 [M, I/128]) - the
    same bytes and scales as ``swiglu_per_token_cast_to_fp8(m_grouped_fp8_block_scaled(a, w13))``.
    ``masked_stride`` > 0: masked row layout (``masked_stride`` rows per group, the first
    ``size_per_group[g]`` valid; other rows of the results are left unwritten)."""
    a8, a_s, b8, b_s, m, n, k, g = _check_pairs(a, b_interleaved)
    assert n % 256 == 0, "n = 2 x intermediate size must be a multiple of 256"
    _lib.require_cuda(size_per_group)
    sizes, is64 = _lib.sizes_arg(size_per_group)
    num_groups = size_per_group.numel()
    if group_to_b is not None:
        assert group_to_b.dtype == torch.int32 and group_to_b.is_contiguous() and group_to_b.numel() == num_groups
        _lib.require_cuda(group_to_b)
    else:
        assert num_groups == g
    if masked_stride:
        assert m == num_groups * masked_stride, "a must hold masked_stride rows per group"
    inter = n // 2
    act = torch.empty((m, inter), device=a8.device, dtype=torch.float8_e4m3fn)
    act_scale = torch.empty((m, inter // 128), device=a8.device, dtype=torch.float32)
    with torch.cuda.device(a8.device):
        rc = _lib.load().b200gemm_fp8_m_grouped_block_swiglu(
            _lib.ptr(a8), _lib.ptr(a_s), _lib.ptr(b8), _lib.ptr(b_s), _lib.ptr(act), _lib.ptr(act_scale), _lib.ptr(sizes),
            is64, num_groups, _lib.ptr(group_to_b) if group_to_b is not None else None, g, m, int(masked_stride), n, k,
            int(num_sms), _lib.stream_ptr(a8.device))
    _lib.check(rc, "b200gemm_fp8_m_grouped_block_swiglu")
    return act, act_scale
