"""Seeded random-shape sweep of the GEMM families against the CPU oracle.

The fixed cases of the other test files pin known-answer tiles, the reference's fixtures and the
benchmark sizes; this file walks through shapes nobody chose: ragged group sizes with empty groups,
N and K that are not multiples of any tile dimension (only of the 16-byte TMA alignment), both
operand layouts, int32 / int64 sizes, every kernel form (tile width, CTA pair on / off / auto).
Tolerances as in the fixed tests: rdiff = sum|a-b| / sum|b| against the oracle's fp32-accumulated,
once-rounded result - 2e-4 for the 16-bit kernels, 5e-4 for the FP8 kernels."""

import random

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.gemm.BF16.k_grouped_gemm_TMA import k_grouped_gemm
from triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_masked_TMA import m_grouped_gemm_masked
from triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_TMA import _m_grouped_gemm_launch
from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_block_scaled import m_grouped_fp8_block_scaled
from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_channel_expert import gmm_fp8_act_per_channel_w_per_expert

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _reset_tuning():
    yield
    _lib.load().b200gemm_set_block_n(0)
    _lib.load().b200gemm_set_cta_pair(-1)
    assert _lib.device_status() == 0


def _ragged_sizes(rng, groups, top):
    """Group sizes in [0, top] with some empty groups and some exact tile multiples."""
    out = []
    for _ in range(groups):
        kind = rng.random()
        if kind < 0.15:
            out.append(0)
        elif kind < 0.3:
            out.append(128 * rng.randint(1, max(1, top // 128)))
        else:
            out.append(rng.randint(1, top))
    if sum(out) == 0:
        out[0] = 1
    return out


@pytest.mark.parametrize("seed", range(12))
def test_m_grouped_16bit(seed):
    rng = random.Random(1000 + seed)
    g = rng.randint(1, 9)
    sizes = _ragged_sizes(rng, g, 700)
    n, k = 8 * rng.randint(1, 80), 8 * rng.randint(1, 70)
    trans_b = rng.random() < 0.5
    dtype = torch.bfloat16 if rng.random() < 0.7 else torch.float16
    size_dtype = torch.int64 if rng.random() < 0.5 else torch.int32
    _lib.load().b200gemm_set_block_n(rng.choice([0, 0, 64, 128, 256]))
    _lib.load().b200gemm_set_cta_pair(rng.choice([-1, 0, 1]))
    gen = torch.Generator().manual_seed(seed)
    m = sum(sizes)
    a = (torch.randn(m + 5, k, generator=gen) * 0.3).to(dtype)
    b = (torch.randn(g, n, k, generator=gen) * 0.3).to(dtype)
    if not trans_b:
        b = b.transpose(1, 2).contiguous()
    ref = O.m_grouped_ref(a[:m], b, sizes, trans_b)
    c = torch.full((m + 5, n), float("nan"), device=DEV, dtype=dtype)
    _m_grouped_gemm_launch(a.to(DEV), b.to(DEV), c, torch.tensor(sizes, dtype=size_dtype, device=DEV), trans_b)
    c = c.cpu()
    assert not torch.isnan(c[:m].float()).any() and torch.isnan(c[m:].float()).all()
    assert O.rdiff(c[:m].float(), ref.float()) < 2e-4, (sizes, n, k, trans_b, dtype)


@pytest.mark.parametrize("seed", range(6))
def test_masked_16bit(seed):
    rng = random.Random(2000 + seed)
    g, e = rng.randint(1, 6), 128 * rng.randint(1, 4)
    masked = [rng.choice([0, e, rng.randint(0, e)]) for _ in range(g)]
    n, k = 8 * rng.randint(1, 60), 8 * rng.randint(1, 60)
    _lib.load().b200gemm_set_cta_pair(rng.choice([-1, 0, 1]))
    gen = torch.Generator().manual_seed(seed)
    lhs = (torch.randn(g * e, k, generator=gen) * 0.3).bfloat16()
    rhs = (torch.randn(g, n, k, generator=gen) * 0.3).bfloat16()
    out0 = torch.full((g * e, n), 7.0, dtype=torch.bfloat16)
    ref = O.m_grouped_masked_ref(lhs, rhs, out0.clone(), masked, e)
    out = out0.clone().to(DEV)
    m_grouped_gemm_masked(lhs.to(DEV), rhs.to(DEV), out, torch.tensor(masked, device=DEV), e)
    out = out.cpu()
    for i, mm in enumerate(masked):
        assert torch.all(out[i * e + mm:(i + 1) * e] == 7.0), "rows past masked_m were written"
    assert O.rdiff(out.float(), ref.float()) < 2e-4, (masked, e, n, k)


@pytest.mark.parametrize("seed", range(8))
def test_k_grouped_16bit(seed):
    rng = random.Random(3000 + seed)
    g = rng.randint(1, 7)
    sizes = _ragged_sizes(rng, g, 900)
    m_dim, n_dim = 8 * rng.randint(1, 50), 8 * rng.randint(1, 50)
    _lib.load().b200gemm_set_cta_pair(rng.choice([-1, 0, 1]))
    gen = torch.Generator().manual_seed(seed)
    k_tot = sum(sizes)
    a = (torch.randn(k_tot + 3, m_dim, generator=gen) * 0.5).bfloat16()
    b = (torch.randn(k_tot + 3, n_dim, generator=gen) * 0.5).bfloat16()
    ref = O.k_grouped_ref(a[:k_tot], b[:k_tot], sizes, fp32_accumulate_explicit=True)
    out = k_grouped_gemm(a.to(DEV), b.to(DEV), torch.tensor(sizes, device=DEV)).cpu()
    assert not torch.isnan(out.float()).any()
    assert O.rdiff(out.float(), ref.float()) < 2e-4, (sizes, m_dim, n_dim)
    for i, s in enumerate(sizes):
        if s == 0:
            assert torch.all(out[i] == 0)


@pytest.mark.parametrize("seed", range(8))
def test_m_grouped_fp8_block_scaled(seed):
    rng = random.Random(4000 + seed)
    g = rng.randint(1, 6)
    sizes = _ragged_sizes(rng, g, 600)
    n, k = 8 * rng.randint(1, 70), 128 * rng.randint(1, 6)
    _lib.load().b200gemm_set_cta_pair(rng.choice([-1, 0, 1]))
    gen = torch.Generator().manual_seed(seed)
    m = sum(sizes)
    x = torch.randn(m + 2, k, generator=gen).bfloat16()
    w = (torch.randn(g, (n + 127) // 128 * 128, k, generator=gen) * 0.05).bfloat16()
    a8, a_s = O.per_token_cast_to_fp8(x)
    qs = [O.per_block_cast_to_fp8(w[i]) for i in range(g)]
    b8_full, b_s = torch.stack([q for q, _ in qs]), torch.stack([s for _, s in qs])
    ref = O.fp8_block_m_grouped_ref(a8[:m], a_s[:m], b8_full, b_s, sizes)[:, :n]
    out = torch.full((m + 2, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    m_grouped_fp8_block_scaled((a8.to(DEV), a_s.to(DEV)), (b8_full[:, :n].contiguous().to(DEV), b_s.to(DEV)),
                               torch.tensor(sizes, device=DEV), out=out)
    out = out.cpu()
    assert not torch.isnan(out[:m].float()).any() and torch.isnan(out[m:].float()).all()
    assert O.rdiff(out[:m].float(), ref.float()) < 5e-4, (sizes, n, k)


@pytest.mark.parametrize("seed", range(6))
def test_m_grouped_fp8_row_channel(seed):
    rng = random.Random(5000 + seed)
    g = rng.randint(1, 6)
    sizes = _ragged_sizes(rng, g, 500)
    n, k = 16 * rng.randint(1, 40), 16 * rng.randint(1, 40)
    dt_a = rng.choice([torch.float8_e4m3fn, torch.float8_e5m2])
    dtype_out = rng.choice([torch.float16, torch.bfloat16])
    _lib.load().b200gemm_set_cta_pair(rng.choice([-1, 0, 1]))
    gen = torch.Generator().manual_seed(seed)
    m = sum(sizes)
    a8 = (torch.randn(m, k, generator=gen) * 50).clamp(-300, 300).to(dt_a)
    b8 = (torch.randn(g, n, k, generator=gen) * 50).clamp(-300, 300).to(torch.float8_e4m3fn)
    a_s = torch.rand(m, generator=gen) * 0.01 + 1e-3
    b_s = torch.rand(g * n, generator=gen) * 0.01 + 1e-3
    ref = O.fp8_rowcol_m_grouped_ref(a8, a_s, b8, b_s, sizes, dtype_out)
    out = gmm_fp8_act_per_channel_w_per_expert(a8.to(DEV), a_s.to(DEV), b8.to(DEV), b_s.to(DEV),
                                               torch.tensor(sizes, device=DEV), dtype_out).cpu()
    assert out.shape == ref.shape and not torch.isnan(out.float()).any()
    assert O.rdiff(out.float(), ref.float()) < 5e-4, (sizes, n, k, dt_a, dtype_out)
