"""Block-scaled FP8 M-grouped / masked GEMM against the CPU oracle (dequantise, fp32 matmul,
one rounding to bf16).  Tolerance rdiff <= 2e-3 (build target); the kernel accumulates the
same products in a different order and multiplies the scales after instead of before the
block sum, so 5e-4 is asserted."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.gemm import deep_gemm_ops
from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_block_scaled import (
    m_grouped_fp8_block_scaled,
    m_grouped_fp8_block_scaled_masked,
)
from triton_grouped_gemm_b200.quant.per_block_cast import per_block_cast_to_fp8, per_token_cast_to_fp8

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 5e-4


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    _lib.load().b200gemm_set_cta_pair(-1)
    assert _lib.device_status() == 0


def _quantised(m, g, n, k, seed):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=gen).bfloat16()
    w = (torch.randn(g, n, k, generator=gen) * 0.02).bfloat16()
    a8, a_s = O.per_token_cast_to_fp8(x)
    qs = [O.per_block_cast_to_fp8(w[i]) for i in range(g)]
    return a8, a_s, torch.stack([q for q, _ in qs]), torch.stack([s for _, s in qs])


def test_single_block_known_answer():
    """One 128x128x128 block with unit scales and small integers: exact."""
    m = n = k = 128
    a = ((torch.arange(m)[:, None] + torch.arange(k)[None, :]) % 5 - 2).float()
    b = ((torch.arange(n)[:, None] * 2 + torch.arange(k)[None, :]) % 7 - 3).float()
    ref = (a @ b.t()) * 0.5 * 0.25
    a8, b8 = a.to(torch.float8_e4m3fn), b.to(torch.float8_e4m3fn)[None].contiguous()
    a_s = torch.full((m, 1), 0.5)
    b_s = torch.full((1, 1, 1), 0.25)
    out = m_grouped_fp8_block_scaled((a8.to(DEV), a_s.to(DEV)), (b8.to(DEV), b_s.to(DEV)),
                                     torch.tensor([m], device=DEV)).cpu()
    assert torch.equal(out.float(), ref.bfloat16().float())


@pytest.mark.parametrize("sizes,n,k", [
    ([128], 128, 128),
    ([128], 256, 256),
    ([300, 0, 1, 127, 129], 384, 512),
    ([5, 700], 3072, 1024),
    ([64, 64], 200, 400),            # n not a multiple of 128, k not a multiple of 128
    ([130] * 30, 512, 384),
])
@pytest.mark.parametrize("pair", [0, 1])
def test_compact_vs_oracle(sizes, n, k, pair):
    _lib.load().b200gemm_set_cta_pair(pair)
    m, g = sum(sizes), len(sizes)
    a8, a_s, b8, b_s = _quantised(m + 3, g, n, (k + 127) // 128 * 128, seed=n + k + g)
    if k % 128:
        a8, b8 = a8[:, :k].contiguous(), b8[:, :, :k].contiguous()
        kpad = a_s.shape[1] * 128
        a_ref = torch.zeros(m + 3, kpad, dtype=a8.dtype)
        a_ref[:, :k] = a8
        b_ref = torch.zeros(g, (n + 127) // 128 * 128, kpad, dtype=b8.dtype)
        b_ref[:, :n, :k] = b8
    else:
        a_ref = a8
        b_ref = torch.zeros(g, (n + 127) // 128 * 128, k, dtype=b8.dtype)
        b_ref[:, :n] = b8
    ref = O.fp8_block_m_grouped_ref(a_ref[:m], a_s[:m], b_ref, b_s, sizes)[:, :n]
    out = torch.full((m + 3, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    m_grouped_fp8_block_scaled((a8.to(DEV), a_s.to(DEV)), (b8.to(DEV), b_s.to(DEV)),
                               torch.tensor(sizes, device=DEV), out=out)
    out = out.cpu()
    assert not torch.isnan(out[:m].float()).any()
    assert torch.isnan(out[m:].float()).all()
    assert O.rdiff(out[:m].float(), ref.float()) < TOL


def test_gpu_quantisers_feed_the_gemm():
    """bf16 -> GPU quantisers -> GPU GEMM equals the all-oracle pipeline."""
    sizes = [200, 56, 384]
    m, g, n, k = sum(sizes), 3, 512, 768
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(m, k, generator=gen).bfloat16()
    w = (torch.randn(g, n, k, generator=gen) * 0.02).bfloat16()
    a = per_token_cast_to_fp8(x.to(DEV))
    b = per_block_cast_to_fp8(w.to(DEV))
    out = m_grouped_fp8_block_scaled(a, b, torch.tensor(sizes, device=DEV)).cpu()
    a8, a_s = O.per_token_cast_to_fp8(x)
    qs = [O.per_block_cast_to_fp8(w[i]) for i in range(g)]
    ref = O.fp8_block_m_grouped_ref(a8, a_s, torch.stack([q for q, _ in qs]), torch.stack([s for _, s in qs]), sizes)
    assert O.rdiff(out.float(), ref.float()) < TOL
    # and close to the unquantised product (fp8 quantisation noise only)
    full = O.m_grouped_ref(x, w, sizes, True).float()
    assert O.rdiff(out.float(), full) < 0.06


@pytest.mark.parametrize("g,e,n,k", [(16, 256, 3072, 512), (4, 128, 128, 256), (3, 384, 640, 384)])
@pytest.mark.parametrize("pair", [0, 1])
def test_masked_vs_oracle(g, e, n, k, pair):
    _lib.load().b200gemm_set_cta_pair(pair)
    a8, a_s, b8, b_s = _quantised(g * e, g, n, k, seed=g + e)
    gen = torch.Generator().manual_seed(e)
    masked = torch.randint(0, e + 1, (g,), generator=gen)
    masked[0] = e
    if g > 2:
        masked[1] = 0
    init = torch.full((g * e, n), 3.0, dtype=torch.bfloat16)
    ref = O.fp8_block_m_grouped_masked_ref(a8, a_s, b8, b_s, init, masked, e)
    out = init.clone().to(DEV)
    assert m_grouped_fp8_block_scaled_masked((a8.to(DEV), a_s.to(DEV)), (b8.to(DEV), b_s.to(DEV)), out,
                                             masked.to(DEV), e) is None
    out = out.cpu()
    assert O.rdiff(out.float(), ref.float()) < TOL
    untouched = torch.ones(g * e, dtype=torch.bool)
    for i, m in enumerate(masked.tolist()):
        untouched[i * e:i * e + m] = False
    assert torch.all(out[untouched] == 3.0)


def test_deep_gemm_ops_padded_layout():
    """The reference's wrapper contract (gemm/deep_gemm_ops.py:60-100): A holds padded rows."""
    sizes = [130, 5, 256]
    padded = [256, 128, 256]
    g, n, k = 3, 256, 256
    a8, a_s, b8, b_s = _quantised(sum(padded), g, n, k, seed=4)
    st = torch.tensor(sizes, device=DEV)
    out = torch.full((sum(padded), n), 9.0, dtype=torch.bfloat16, device=DEV)
    res = deep_gemm_ops.m_grouped_fp8_nt_contiguous((a8.to(DEV), a_s.to(DEV)), (b8.to(DEV), b_s.to(DEV)), st, out=out)
    assert res.data_ptr() == out.data_ptr()
    out = out.cpu()
    row = 0
    for i, (s, p) in enumerate(zip(sizes, padded)):
        ref = O.fp8_block_m_grouped_ref(a8[row:row + s], a_s[row:row + s], b8[i:i + 1], b_s[i:i + 1], [s])
        assert O.rdiff(out[row:row + s].float(), ref.float()) < TOL
        assert torch.all(out[row + s:row + p] == 9.0)
        row += p
    with pytest.raises(ValueError, match="A must include padded expert rows"):
        deep_gemm_ops.m_grouped_fp8_nt_contiguous((a8[:-128].to(DEV), a_s[:-128].to(DEV)),
                                                  (b8.to(DEV), b_s.to(DEV)), st)
    # bf16 twin
    gen = torch.Generator().manual_seed(1)
    a = torch.randn(sum(padded), k, generator=gen).bfloat16()
    b = torch.randn(g, n, k, generator=gen).bfloat16()
    o = torch.full((sum(padded), n), 9.0, dtype=torch.bfloat16, device=DEV)
    deep_gemm_ops.m_grouped_bf16_nt_contiguous(a.to(DEV), b.to(DEV), st, out=o)
    o = o.cpu()
    row = 0
    for i, (s, p) in enumerate(zip(sizes, padded)):
        ref = (a[row:row + s].float() @ b[i].float().t()).bfloat16()
        assert O.rdiff(o[row:row + s].float(), ref.float()) < 2e-4
        assert torch.all(o[row + s:row + p] == 9.0)
        row += p


def test_full_size_properties():
    """Benchmark size (G=128, ~663k rows, K=4096, N=3072): sampled rows against the oracle and
    exact linearity in the weight scales over the whole output."""
    sizes = O.routing_sizes(128, 655360, seed=2026)
    m = int(sizes.sum())
    gen = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(m, 4096, device=DEV, generator=gen, dtype=torch.bfloat16)
    w = (torch.randn(128, 3072, 4096, device=DEV, generator=gen, dtype=torch.bfloat16) * 0.02)
    a = per_token_cast_to_fp8(x)
    b = per_block_cast_to_fp8(w)
    del x, w
    sz = sizes.to(DEV)
    c1 = m_grouped_fp8_block_scaled(a, b, sz)
    c2 = m_grouped_fp8_block_scaled(a, (b[0], b[1] * 2), sz)
    assert torch.equal(c1 * 2, c2)
    starts = torch.cumsum(sizes, 0) - sizes
    # every group against real arithmetic: its first, a middle and its last rows (8 each)
    for g in range(128):
        s0, sz_g = int(starts[g]), int(sizes[g])
        rows = (torch.cat([torch.arange(0, 8), torch.arange(sz_g // 2, sz_g // 2 + 8), torch.arange(sz_g - 8, sz_g)])
                + s0).to(DEV)
        ref = O.fp8_block_m_grouped_ref(a[0][rows].cpu(), a[1][rows].cpu(), b[0][g:g + 1].cpu(), b[1][g:g + 1].cpu(),
                                        [rows.numel()])
        assert O.rdiff(c1[rows].float().cpu(), ref.float()) < TOL, f"group {g}"
    for g in (0, 64, 127):
        s = int(starts[g])
        rows = 64
        ref = O.fp8_block_m_grouped_ref(a[0][s:s + rows].cpu(), a[1][s:s + rows].cpu(), b[0][g:g + 1].cpu(),
                                        b[1][g:g + 1].cpu(), [rows])
        assert O.rdiff(c1[s:s + rows].float().cpu(), ref.float()) < TOL


@pytest.mark.parametrize("pair", [0, 1])
def test_group_to_weight_map(pair):
    """Row blocks in arbitrary order, each mapped to one of the weight matrices (the layout an
    all-to-all delivers: [source rank][expert] blocks).  Same result as gathering every
    expert's rows together first."""
    _lib.load().b200gemm_set_cta_pair(pair)
    n, k, num_b = 384, 512, 3
    block_sizes = [70, 0, 300, 129, 5, 0, 256, 33]        # 8 blocks
    block_expert = [0, 1, 2, 0, 1, 2, 2, 0]
    m = sum(block_sizes)
    a8, a_s, b8, b_s = _quantised(m, num_b, n, k, seed=17)
    out = m_grouped_fp8_block_scaled((a8.to(DEV), a_s.to(DEV)), (b8.to(DEV), b_s.to(DEV)),
                                     torch.tensor(block_sizes, device=DEV),
                                     group_to_b=torch.tensor(block_expert, dtype=torch.int32, device=DEV)).cpu()
    # oracle: treat every block as a group of its own with a copy of its expert's weights
    b8_blocks = torch.stack([b8[e] for e in block_expert])
    b_s_blocks = torch.stack([b_s[e] for e in block_expert])
    ref = O.fp8_block_m_grouped_ref(a8, a_s, b8_blocks, b_s_blocks, block_sizes)
    assert O.rdiff(out.float(), ref.float()) < 5e-4
    # identical bits to the unmapped kernel on the expanded weights
    out2 = m_grouped_fp8_block_scaled((a8.to(DEV), a_s.to(DEV)), (b8_blocks.to(DEV), b_s_blocks.to(DEV)),
                                      torch.tensor(block_sizes, device=DEV)).cpu()
    assert torch.equal(out, out2)


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("sizes,inter,k", [([300, 0, 1, 127, 129], 256, 512), ([128], 128, 128), ([64, 700, 5], 384, 1024)])
def test_swiglu_epilogue_is_bit_identical_to_product_plus_quantiser(sizes, inter, k, pair):
    """Gate+up GEMM with SwiGLU + 1x128 quantiser in its epilogue (weights interleaved in 128-row
    blocks) against the bf16 product followed by the SwiGLU quantiser kernel: same bytes, same
    scales; also with row blocks mapped to weights."""
    from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_block_scaled import (interleave_gate_up,
                                                                              m_grouped_fp8_block_scaled_swiglu)
    from triton_grouped_gemm_b200.quant.per_block_cast import (per_block_cast_to_fp8, per_token_cast_to_fp8,
                                                             swiglu_per_token_cast_to_fp8)

    _lib.load().b200gemm_set_cta_pair(pair)
    g, m = len(sizes), sum(sizes)
    gen = torch.Generator().manual_seed(inter + k + g)
    x = torch.randn(m, k, generator=gen).bfloat16().to(DEV)
    w13 = (torch.randn(g, 2 * inter, k, generator=gen) * 0.05).bfloat16().to(DEV)
    st = torch.tensor(sizes, device=DEV)
    a = per_token_cast_to_fp8(x)
    h = m_grouped_fp8_block_scaled(a, per_block_cast_to_fp8(w13), st)
    q_ref, s_ref = swiglu_per_token_cast_to_fp8(h)
    q, s = m_grouped_fp8_block_scaled_swiglu(a, per_block_cast_to_fp8(interleave_gate_up(w13)), st)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s, s_ref)
    # masked layout: 2 slots per group... every group gets a slot of `stride` rows, first sizes[g] valid
    stride = 768
    xm = torch.zeros(g * stride, k, dtype=torch.bfloat16, device=DEV)
    row = 0
    for i, n_i in enumerate(sizes):
        xm[i * stride:i * stride + n_i] = x[row:row + n_i]
        row += n_i
    am = per_token_cast_to_fp8(xm)
    qm, sm = m_grouped_fp8_block_scaled_swiglu(am, per_block_cast_to_fp8(interleave_gate_up(w13)), st, masked_stride=stride)
    row = 0
    for i, n_i in enumerate(sizes):
        assert torch.equal(qm[i * stride:i * stride + n_i].view(torch.uint8), q_ref[row:row + n_i].view(torch.uint8))
        assert torch.equal(sm[i * stride:i * stride + n_i], s_ref[row:row + n_i])
        row += n_i


@pytest.mark.parametrize("pair", [0, 1])
def test_sizes_summing_past_m_rows_are_cut_off_and_flagged(pair):
    """sum(sizes) > m_rows: the overrunning group is cut at m_rows, nothing past the end of c is
    written (c is a prefix of a larger buffer of this test, so an overrun would show instead of
    faulting), the activation scales are not indexed there, and status bit 0x10 is raised."""
    _lib.load().b200gemm_set_cta_pair(pair)
    sizes_bad, m_rows, n, k = [100, 300, 200], 350, 512, 384
    a8, a_s, b8, b_s = _quantised(m_rows, 3, n, k, seed=31)
    c_big = torch.full((m_rows + 512, n), 5.0, device=DEV, dtype=torch.bfloat16)
    m_grouped_fp8_block_scaled((a8.to(DEV), a_s.to(DEV)), (b8.to(DEV), b_s.to(DEV)),
                               torch.tensor(sizes_bad, device=DEV), out=c_big[:m_rows])
    assert _lib.device_status() == 0x10
    out = c_big.cpu()
    assert torch.all(out[m_rows:] == 5.0)
    ref = O.fp8_block_m_grouped_ref(a8, a_s, b8, b_s, [100, 250, 0])
    assert O.rdiff(out[:m_rows].float(), ref.float()) < TOL
