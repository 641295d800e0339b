"""Block-scaled FP8 MoE feed-forward layer with expert parallelism, on the B200 kernels.

Per rank: quantise local tokens 1x128 -> dispatch fp8 rows + scales to the expert owners
(all-to-all) -> gate+up grouped GEMM (fp8, block scaled) -> SwiGLU fused with 1x128
re-quantisation -> down grouped GEMM -> combine (all-to-all back, router-weighted sum).
Weights are quantised 128x128 once at construction.  A decode variant runs the two GEMMs on
the masked layout ([local experts, m_max] slots, ``masked_m`` valid rows each).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..gemm.FP8.m_grouped_gemm_block_scaled import m_grouped_fp8_block_scaled, m_grouped_fp8_block_scaled_masked
from ..quant.per_block_cast import per_block_cast_to_fp8, per_token_cast_to_fp8, swiglu_per_token_cast_to_fp8
from .dispatch import combine, dispatch, make_plan


class Fp8MoELayer:
    def __init__(self, w13: torch.Tensor, w2: torch.Tensor, num_experts: int,
                 group: Optional[dist.ProcessGroup] = None):
        """w13 [E_local, 2*I, H] (gate rows then up rows), w2 [E_local, H, I], bf16, this rank's experts."""
        assert w13.dim() == 3 and w2.dim() == 3 and w13.shape[0] == w2.shape[0]
        self.group = group
        self.num_experts = num_experts
        self.e_local, two_i, self.hidden = w13.shape
        self.inter = two_i // 2
        assert w2.shape == (self.e_local, self.hidden, self.inter)
        self.w13 = per_block_cast_to_fp8(w13.contiguous())
        self.w2 = per_block_cast_to_fp8(w2.contiguous())

    def experts(self, x8: torch.Tensor, xs: torch.Tensor, size_per_group: torch.Tensor) -> torch.Tensor:
        """Rows already grouped by local expert: [R, H] fp8 + scales -> [R, H] bf16."""
        h = m_grouped_fp8_block_scaled((x8, xs), self.w13, size_per_group)
        a8, a_s = swiglu_per_token_cast_to_fp8(h)
        return m_grouped_fp8_block_scaled((a8, a_s), self.w2, size_per_group)

    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weight: torch.Tensor) -> torch.Tensor:
        """x [T, H] bf16, topk_idx/topk_weight [T, k] -> [T, H] bf16."""
        x8, xs = per_token_cast_to_fp8(x.contiguous())
        plan = make_plan(topk_idx, self.num_experts, self.group)
        r8 = dispatch(plan, x8, self.group)
        rs = dispatch(plan, xs, self.group)
        y = self.experts(r8.contiguous(), rs.contiguous(), plan.size_per_group)
        return combine(plan, y, topk_weight, self.group)

    def decode(self, x8: torch.Tensor, xs: torch.Tensor, masked_m: torch.Tensor, m_max: int,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Masked layout: x8 [E_local*m_max, H] fp8 + scales, ``masked_m`` valid rows per expert.
        Rows past ``masked_m[e]`` of each slot are left as they were in ``out`` (zeros if None)."""
        rows = self.e_local * m_max
        assert x8.shape == (rows, self.hidden)
        h = torch.zeros((rows, 2 * self.inter), device=x8.device, dtype=torch.bfloat16)
        m_grouped_fp8_block_scaled_masked((x8, xs), self.w13, h, masked_m, m_max)
        a8, a_s = swiglu_per_token_cast_to_fp8(h)
        if out is None:
            out = torch.zeros((rows, self.hidden), device=x8.device, dtype=torch.bfloat16)
        m_grouped_fp8_block_scaled_masked((a8, a_s), self.w2, out, masked_m, m_max)
        return out


def synthetic_routing(num_tokens: int, num_experts: int, top_k: int, seed: int,
                      device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """Router of the benchmark configuration: logits ~ N(0, 0.5), softmax, top-k (weights
    renormalised over the selected experts)."""
    gen = torch.Generator().manual_seed(seed)
    logits = 0.5 * torch.randn(num_tokens, num_experts, generator=gen)
    p = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(p, top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    return idx.to(device), w.to(device)
