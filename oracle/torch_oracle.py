"""CPU restatement (torch, host cores) of the reference algorithms on the hot path.

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.

Every function names the reference source it follows (paths are relative to the
root of DeepLink-org/Triton_Grouped_GEMM).  The restatements are pinned by
``tests/golden/*.pt``: fixtures produced by importing / executing the
reference's own torch functions (``tests/golden/make_golden.py``), checked by
``tests/test_oracle_golden.py``.

One boundary is unpinned: the block-scaled FP8 grouped GEMM (1x128 activation
scales, 128x128 weight scales).  The reference only forwards that call to the
external ``deep_gemm`` package (gemm/deep_gemm_ops.py:60-100; lazy import, no
version pin, not vendored, never exercised by the reference's tests), so
``fp8_block_m_grouped_ref`` below restates the published contract
(dequantise, accumulate in fp32, round once to bf16) -- parity unpinned for that
one function; its inputs come from the pinned quantisers.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

__all__ = [
    "rdiff",
    "row_max_normalization",
    "ceil_div",
    "m_grouped_ref",
    "m_grouped_masked_ref",
    "k_grouped_ref",
    "per_token_cast_to_fp8",
    "per_block_cast_to_fp8",
    "per_channel_cast_to_fp8",
    "per_expert_cast_to_fp8",
    "trans_quant_expand_ref",
    "fp8_rowcol_m_grouped_ref",
    "fp8_rowcol_k_grouped_ref",
    "fp8_block_m_grouped_ref",
    "fp8_block_m_grouped_masked_ref",
    "fp8_block_k_grouped_ref",
    "dequant_1x128",
    "dequant_128x128",
    "layout_round_up",
    "layout_group_starts",
    "layout_grouped",
    "layout_psum",
    "layout_m_grouped_metadata",
    "routing_sizes",
    "config0_inputs",
    "moe_layer_ref",
]


# --------------------------------------------------------------------------- metrics

def rdiff(a: torch.Tensor, b: torch.Tensor) -> float:
    """sum|a-b| / sum|b| with b the oracle (the tolerance metric of the build target)."""
    a = a.double()
    b = b.double()
    den = b.abs().sum().item()
    num = (a - b).abs().sum().item()
    if den == 0.0:
        return 0.0 if num == 0.0 else float("inf")
    return num / den


def row_max_normalization(t: torch.Tensor) -> torch.Tensor:
    """gemm/BF16/utils.py:41-44 -- divide each row by (max|row| + 1e-9)."""
    m = t.abs().max(dim=-1).values + 1e-9
    return t / m.unsqueeze(-1)


def ceil_div(x: int, y: int) -> int:
    return (x + y - 1) // y


def _sizes_list(sizes) -> List[int]:
    if isinstance(sizes, torch.Tensor):
        return [int(v) for v in sizes.detach().cpu().tolist()]
    return [int(v) for v in sizes]


# --------------------------------------------------------------------------- BF16 GEMMs

def m_grouped_ref(a: torch.Tensor, b: torch.Tensor, sizes, trans_b: bool,
                  fp32_accumulate_explicit: bool = False) -> torch.Tensor:
    """Per-group ``a[rows of g] @ B_g`` (gemm/BF16/utils.py:5-14,
    gemm/BF16/m_grouped_gemm_TMA.py:573-581).

    ``trans_b=True``: ``b`` is [G, N, K]; else [G, K, N].  The reference multiplies
    the 16-bit tensors directly (fp32 accumulation inside the BLAS, one rounding to
    the input dtype).  ``fp32_accumulate_explicit`` upcasts first and rounds the
    fp32 product once; the two agree up to accumulation order.
    """
    out = []
    start = 0
    for g, size in enumerate(_sizes_list(sizes)):
        rhs = b[g].t() if trans_b else b[g]
        lhs = a[start:start + size]
        if fp32_accumulate_explicit:
            out.append((lhs.float() @ rhs.float()).to(a.dtype))
        else:
            out.append(lhs @ rhs)
        start += size
    if not out:
        n = b.shape[1] if trans_b else b.shape[2]
        return a.new_empty(0, n)
    return torch.cat(out).contiguous()


def m_grouped_masked_ref(lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor,
                         masked_m, expected_m: int,
                         fp32_accumulate_explicit: bool = False) -> torch.Tensor:
    """Masked layout (gemm/BF16/m_grouped_gemm_masked_TMA.py:104-134,164-250).

    ``lhs`` [G*E, K], ``rhs`` [G, N, K], ``out`` [G*E, N].  For each group only the
    first ``masked_m[g]`` rows starting at row ``g*E`` are written; the other rows of
    ``out`` keep whatever they held.  Returns a new tensor (``out`` is not mutated).
    """
    res = out.clone()
    for g, m in enumerate(_sizes_list(masked_m)):
        r0 = g * expected_m
        a = lhs[r0:r0 + m]
        w = rhs[g].t()
        if fp32_accumulate_explicit:
            res[r0:r0 + m] = (a.float() @ w.float()).to(out.dtype)
        else:
            res[r0:r0 + m] = (a @ w).to(out.dtype)
    return res


def k_grouped_ref(a: torch.Tensor, b: torch.Tensor, sizes,
                  fp32_accumulate_explicit: bool = False) -> torch.Tensor:
    """``C[g] = A[gs:ge].T @ B[gs:ge]`` (gemm/BF16/k_grouped_gemm_TMA.py:402-416).

    ``a`` [K_total, M_DIM], ``b`` [K_total, N_DIM] -> [G, M_DIM, N_DIM].  An empty
    group gives a zero matrix (the TMA kernel stores its zero accumulator,
    gemm/BF16/k_grouped_gemm_TMA.py:141,167-170).
    """
    sz = _sizes_list(sizes)
    out = a.new_zeros(len(sz), a.shape[1], b.shape[1])
    start = 0
    for g, size in enumerate(sz):
        lhs = a[start:start + size]
        rhs = b[start:start + size]
        if size:
            if fp32_accumulate_explicit:
                out[g] = (lhs.float().t() @ rhs.float()).to(a.dtype)
            else:
                out[g] = lhs.t() @ rhs
        start += size
    return out.contiguous()


# --------------------------------------------------------------------------- FP8 casts

def per_token_cast_to_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """1x128 activation quantiser (gemm/FP8/m_grouped_gemm_channel_expert.py:217-222).

    amax over each 128-wide K block (taken on the 16-bit values, widened to fp32,
    clamped below at 1e-4); q = fp32(x) * (448 / amax) cast to e4m3 (round to
    nearest even); scale = amax / 448.  NOTE: ``448.0 / tensor`` is evaluated by torch as
    ``tensor.reciprocal() * 448.0`` (two roundings) -- kept verbatim here because it
    decides bytes; ``tensor / 448.0`` is a true division on the host.
    """
    assert x.dim() == 2 and x.size(1) % 128 == 0
    m, n = x.shape
    v = x.view(m, -1, 128)
    amax = v.abs().float().amax(dim=2).view(m, -1).clamp(1e-4)
    q = (v * (448.0 / amax.unsqueeze(2))).to(torch.float8_e4m3fn).view(m, n)
    return q, (amax / 448.0).view(m, -1)


def per_block_cast_to_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """128x128 weight quantiser (gemm/FP8/m_grouped_gemm_channel_expert.py:237-245).

    Zero-pads to multiples of 128 in both dims, one amax per 128x128 block (clamped
    below at 1e-4), q = fp32(x) * (448 / amax) -> e4m3; returns q[:m,:n] and scales
    [ceil(m/128), ceil(n/128)].
    """
    assert x.dim() == 2
    m, n = x.shape
    xp = torch.zeros((ceil_div(m, 128) * 128, ceil_div(n, 128) * 128), dtype=x.dtype, device=x.device)
    xp[:m, :n] = x
    v = xp.view(-1, 128, xp.size(1) // 128, 128)
    amax = v.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    q = (v * (448.0 / amax)).to(torch.float8_e4m3fn)
    return q.view_as(xp)[:m, :n].contiguous(), (amax / 448.0).view(v.size(0), v.size(2))


def per_channel_cast_to_fp8(x: torch.Tensor, dtype=torch.float8_e4m3fn) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scale per row over the whole row
    (gemm/FP8/m_grouped_gemm_channel_expert.py:224-234)."""
    assert x.dim() == 2 and x.size(1) % 128 == 0
    m, n = x.shape
    v = x.view(m, -1, n)
    amax = v.abs().float().amax(dim=2).view(m, -1).clamp(1e-4)
    fmax = torch.finfo(dtype).max
    return (v * (fmax / amax.unsqueeze(2))).to(dtype).view(m, n), (amax / fmax).view(m, -1)


def per_expert_cast_to_fp8(x: torch.Tensor, dtype=torch.float8_e4m3fn) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scale per expert over its whole [m, n] matrix
    (gemm/FP8/m_grouped_gemm_channel_expert.py:247-261).  Requires m, n multiples of
    128 (the reference views a padded copy with the unpadded shape)."""
    assert x.dim() == 3
    g, m, n = x.shape
    assert m % 128 == 0 and n % 128 == 0
    v = x.reshape(g, m, 1, n)
    amax = v.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    fmax = torch.finfo(dtype).max
    q = (v * (fmax / amax)).to(dtype)
    return q.view(g, m, n).contiguous(), (amax / fmax).view(g, 1)


def _to_fp8_saturated(x: torch.Tensor, dtype) -> torch.Tensor:
    """quant/trans_per_block_quant_expand_128x.py:216-219."""
    mx = torch.finfo(dtype).max
    return x.clamp(min=-mx, max=mx).to(dtype)


def _trans_quant_one_expert(x: torch.Tensor, block: int = 128, dtype=torch.float8_e4m3fn, clamp_scale: bool = True):
    """quant/trans_per_block_quant_expand_128x.py:222-250 -- one expert:
    transpose [seq, dim] -> [dim, seq], zero-pad seq to a multiple of 128, one
    scale = amax/448 per 128x128 block, q = clamp(fp32(x)/scale).  ``clamp_scale`` adds the
    clamp of the scale to [1e-12, 3e38] that the reference's shipped operator applies (its
    Triton kernel, same file :124-126); without it this is the torch helper alone, whose
    all-zero block gives scale 0 and NaN bytes."""
    x = x.T
    dim, seq = x.shape
    seq_e = ceil_div(seq, block) * block
    xe = torch.cat([x, x.new_zeros((dim, seq_e - seq))], dim=-1)
    xe = xe.reshape(dim // block, block, seq_e // block, block).transpose(1, 2).reshape(-1, block * block)
    amax = xe.abs().amax(-1, True)
    scale = amax.float() / torch.finfo(dtype).max
    if clamp_scale:
        scale = scale.clamp(min=1e-12, max=3e38)
    q = _to_fp8_saturated(xe / scale, dtype)
    q = q.reshape(dim // block, seq_e // block, block, block).transpose(1, 2).reshape(dim, seq_e)
    return q, scale.reshape(dim // block, seq_e // block)


def trans_quant_expand_ref(x: torch.Tensor, tokens_per_expert,
                           clamp_scale: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Transposing 128x128 quantiser with per-expert expansion
    (quant/trans_per_block_quant_expand_128x.py:253-273).

    ``x`` [M, N] -> fp8 [N, M_EXPAND], scales [N/128, M_EXPAND/128], padded sizes.
    ``M_EXPAND = M + 128*G - M % 128`` (same file :172); columns / scales beyond the
    sum of padded sizes are zero.  With ``clamp_scale`` (the operator's behaviour, see
    ``_trans_quant_one_expert``) an all-zero 128x128 block inside an expert gives zero bytes and
    scale 1e-12; with ``clamp_scale=False`` (the torch helper, which the CPU fixtures were made
    with) it gives scale 0 and NaN bytes (0/0).
    """
    sz = _sizes_list(tokens_per_expert)
    m = x.shape[0]
    ne = len(sz)
    qs, ss = [], []
    for part in torch.split(x, sz, dim=0):
        q, s = _trans_quant_one_expert(part, clamp_scale=clamp_scale)
        qs.append(q)
        ss.append(s)
    q = torch.cat(qs, dim=-1)
    s = torch.cat(ss, dim=-1)
    m_expand = m + 128 * ne - m % 128
    q = torch.cat([q, q.new_zeros((q.shape[0], m_expand - q.shape[1]))], dim=1)
    s = torch.cat([s, s.new_zeros((s.shape[0], m_expand // 128 - s.shape[1]))], dim=1)
    padded = torch.tensor([ceil_div(v, 128) * 128 for v in sz], dtype=torch.int64)
    return q, s, padded


# --------------------------------------------------------------------------- FP8 GEMMs

def fp8_rowcol_m_grouped_ref(a8, a_scale, b8, b_scale, sizes, dtype_out=torch.float16) -> torch.Tensor:
    """gemm/FP8/m_grouped_gemm_channel_expert.py:64-136: fp32 accumulation of the
    fp8 products over the whole K, then ``* a_scale[m] * b_scale[g*N+n]``."""
    g_, n, k = b8.shape
    a_scale = a_scale.reshape(-1).float()
    b_scale = b_scale.reshape(g_, n).float()
    out = torch.empty(a8.shape[0], n, dtype=dtype_out)
    start = 0
    for g, size in enumerate(_sizes_list(sizes)):
        acc = a8[start:start + size].float() @ b8[g].float().t()
        out[start:start + size] = (acc * a_scale[start:start + size, None] * b_scale[g][None, :]).to(dtype_out)
        start += size
    return out


def fp8_rowcol_k_grouped_ref(x8, x_scale, y8, y_scale, tokens_per_expert, m, n, num_groups) -> torch.Tensor:
    """gemm/FP8/k_grouped_gemm_channel_expert.py:64-140.  ``x8`` [M, K_tot],
    ``y8`` [N, K_tot]; ``x_scale``/``y_scale`` are logical [M, G]/[N, G] whose memory is
    group-major (flat index g*M+m, same file :121-124); out[g] = (X_g . Y_g^T) *
    xs[m,g] * ys[n,g] -> bf16 [G, M, N]."""
    xs = x_scale.float()
    ys = y_scale.float()
    out = torch.empty(num_groups, m, n, dtype=torch.bfloat16)
    start = 0
    for g, t in enumerate(_sizes_list(tokens_per_expert)):
        acc = x8[:, start:start + t].float() @ y8[:, start:start + t].float().t()
        out[g] = (acc * xs[:, g][:, None] * ys[:, g][None, :]).to(torch.bfloat16)
        start += t
    return out


def dequant_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """fp32(q[m,k]) * s[m, k//128]."""
    m, k = q.shape
    return (q.float().view(m, k // 128, 128) * s.float().unsqueeze(2)).view(m, k)


def dequant_128x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """fp32(q[n,k]) * s[n//128, k//128] for one expert (n, k multiples of 128)."""
    n, k = q.shape
    return (q.float().view(n // 128, 128, k // 128, 128) * s.float()[:, None, :, None]).reshape(n, k)


def fp8_block_m_grouped_ref(a8, a_s, b8, b_s, sizes) -> torch.Tensor:
    """Block-scaled FP8 M-grouped GEMM contract (gemm/deep_gemm_ops.py:60-100,
    README.md:173-179): C[m,n] = sum_kb (sum_{k in kb} a8*b8) * as[m,kb] * bs[g,n//128,kb],
    fp32 throughout, one rounding to bf16.  PARITY UNPINNED (see module docstring)."""
    g_, n, k = b8.shape
    a = dequant_1x128(a8, a_s)
    out = torch.empty(a8.shape[0], n, dtype=torch.bfloat16)
    start = 0
    for g, size in enumerate(_sizes_list(sizes)):
        w = dequant_128x128(b8[g], b_s[g])
        out[start:start + size] = (a[start:start + size] @ w.t()).to(torch.bfloat16)
        start += size
    return out


def fp8_block_k_grouped_ref(x8, xs, y8, ys, padded_sizes) -> torch.Tensor:
    """Block-scaled FP8 K-grouped GEMM (the FP8 weight gradient) on two outputs of the transposing
    quantiser (quant/trans_per_block_quant_expand_128x.py:135-208): ``x8`` [M_DIM, M_EXPAND],
    ``y8`` [N_DIM, M_EXPAND] with one scale per 128x128 block; expert g owns the tokens after those
    of the experts before it (``padded_sizes``, multiples of 128).  out[g] = dequant(x)[:, tokens
    of g] @ dequant(y)[:, tokens of g]^T in fp32, one rounding to bf16; an expert without tokens
    gives zeros.  PARITY UNPINNED: the reference ships the quantiser but no kernel that consumes
    its output, so there is no reference arithmetic to pin; the contract restated here is the
    dequantised product."""
    xd = dequant_128x128(x8, xs)
    yd = dequant_128x128(y8, ys)
    sz = _sizes_list(padded_sizes)
    out = torch.zeros(len(sz), x8.shape[0], y8.shape[0], dtype=torch.bfloat16)
    start = 0
    for g, size in enumerate(sz):
        if size:
            out[g] = (xd[:, start:start + size] @ yd[:, start:start + size].t()).to(torch.bfloat16)
        start += size
    return out


def fp8_block_m_grouped_masked_ref(a8, a_s, b8, b_s, out, masked_m, expected_m) -> torch.Tensor:
    """Masked-layout twin of ``fp8_block_m_grouped_ref`` (rows g*E .. g*E+masked_m[g])."""
    res = out.clone()
    a = dequant_1x128(a8, a_s)
    for g, m in enumerate(_sizes_list(masked_m)):
        r0 = g * expected_m
        w = dequant_128x128(b8[g], b_s[g])
        res[r0:r0 + m] = (a[r0:r0 + m] @ w.t()).to(out.dtype)
    return res


# --------------------------------------------------------------------------- integer layouts

def layout_round_up(sizes: Sequence[int], alignment: int) -> List[int]:
    """gemm/layout.py:48-51."""
    if alignment <= 0:
        raise ValueError(f"alignment must be positive, got {alignment}")
    return [(int(s) + alignment - 1) // alignment * alignment for s in sizes]


def layout_group_starts(sizes: Sequence[int], padded: bool = False, block_m: int = 128) -> List[int]:
    """gemm/layout.py:61-70 -- exclusive prefix sum of the (optionally padded) sizes."""
    use = layout_round_up(sizes, block_m) if padded else [int(s) for s in sizes]
    out, acc = [], 0
    for s in use:
        out.append(acc)
        acc += s
    return out


def layout_grouped(sizes: Sequence[int], block_m: int = 128) -> List[int]:
    """gemm/layout.py:73-97 -- one entry per padded row: expert id on real rows, -1 on pad rows."""
    out: List[int] = []
    for g, (s, p) in enumerate(zip(sizes, layout_round_up(sizes, block_m))):
        out += [g] * int(s) + [-1] * (p - int(s))
    return out


def layout_psum(sizes: Sequence[int], block_m: int = 128) -> List[int]:
    """gemm/layout.py:100-119 -- actual end offset of each expert in padded coordinates."""
    out, start = [], 0
    for s, p in zip(sizes, layout_round_up(sizes, block_m)):
        out.append(start + int(s))
        start += p
    return out


def layout_m_grouped_metadata(sizes: Sequence[int], block_m: int = 128):
    """gemm/BF16/m_grouped_gemm_TMA.py:297-326 -- (pad_start, pad_end, group_start,
    group_end, m_indices_pad[: total padded tiles], M_pad) as Python lists/ints."""
    p = layout_round_up(sizes, block_m)
    pad_start = layout_group_starts(p)
    pad_end = [a + b for a, b in zip(pad_start, p)]
    group_start = layout_group_starts(sizes)
    group_end = [a + int(b) for a, b in zip(group_start, sizes)]
    m_idx: List[int] = []
    for g, pg in enumerate(p):
        m_idx += [g] * (pg // block_m)
    return pad_start, pad_end, group_start, group_end, m_idx, sum(p)


# --------------------------------------------------------------------------- workload generators

def routing_sizes(num_groups: int, total_rows: int, seed: int = 2026, std: float = 0.5,
                  pad_to: int = 128) -> torch.Tensor:
    """Per-expert row counts for the MoE benchmark shapes: multinomial over
    ``total_rows`` draws with probabilities softmax(N(0, std) logits), each count padded
    up to a multiple of ``pad_to`` (0 = no padding).  Seeded CPU generator -> the same
    sizes everywhere."""
    gen = torch.Generator().manual_seed(seed)
    logits = std * torch.randn(num_groups, generator=gen)
    p = torch.softmax(logits, dim=0)
    draws = torch.multinomial(p, total_rows, replacement=True, generator=gen)
    counts = torch.bincount(draws, minlength=num_groups)
    if pad_to:
        counts = (counts + pad_to - 1) // pad_to * pad_to
    return counts.to(torch.int64)


def config0_inputs(seed: int = 0):
    """The CPU-runnable case: G=4, sizes uniform in [64,256] rounded up to 16,
    K=512, N=256, trans_b=True, A and B ~ N(0,1)*0.1 in bf16."""
    gen = torch.Generator().manual_seed(seed)
    sizes = torch.randint(64, 257, (4,), generator=gen)
    sizes = (sizes + 15) // 16 * 16
    m = int(sizes.sum())
    a = (torch.randn(m, 512, generator=gen) * 0.1).to(torch.bfloat16)
    b = (torch.randn(4, 256, 512, generator=gen) * 0.1).to(torch.bfloat16)
    return a, b, sizes.to(torch.int64)


# --------------------------------------------------------------------------- expert-parallel layer

def moe_layer_ref(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                  w13: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """fp32 restatement of the block-scaled FP8 MoE layer the expert-parallel path runs:
    for every (token, expert) pair: quantise the token 1x128, gate+up GEMM against the
    128x128-quantised ``w13[e]`` ([2I, H]), SiLU(gate)*up, quantise 1x128, down GEMM
    against the quantised ``w2[e]`` ([H, I]), then the top-k weighted sum per token.
    Intermediate tensors are rounded to bf16 exactly where the GPU pipeline stores
    bf16.  Small inputs only (loops over experts)."""
    t, h = x.shape
    e_, two_i, _ = w13.shape
    inter = two_i // 2
    out = torch.zeros(t, h, dtype=torch.float32)
    xq, xs = per_token_cast_to_fp8(x)
    xd = dequant_1x128(xq, xs)
    for e in range(e_):
        tok, slot = (topk_idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        q13, s13 = per_block_cast_to_fp8(w13[e])
        q2, s2 = per_block_cast_to_fp8(w2[e])
        hmid = (xd[tok] @ dequant_128x128(q13, s13).t()).to(torch.bfloat16)
        gate, up = hmid[:, :inter].float(), hmid[:, inter:].float()
        act = (torch.nn.functional.silu(gate) * up).to(torch.bfloat16)
        aq, as_ = per_token_cast_to_fp8(act)
        y = (dequant_1x128(aq, as_) @ dequant_128x128(q2, s2).t()).to(torch.bfloat16)
        out.index_add_(0, tok, y.float() * topk_w[tok, slot].float().unsqueeze(1))
    return out.to(torch.bfloat16)
