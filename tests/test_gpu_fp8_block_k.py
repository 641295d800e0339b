"""Block-scaled FP8 K-grouped GEMM (the FP8 expert weight gradient) against the CPU oracle:
dequantise both quantiser outputs with their 128x128 scales, fp32 product per expert, one
rounding to bf16.  Parity is unpinned by nature - the reference ships the transposing quantiser
but no kernel that consumes its output - so the oracle restates the contract; the operands come
from the quantiser that IS pinned bit for bit.  Tolerance rdiff <= 2e-3 (build target); the
kernel sums the same products in another order and applies the scales per k-block, so 5e-4 is
asserted."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.gemm.FP8.k_grouped_gemm_block_scaled import fp8_wgrad, k_grouped_fp8_block_scaled
from triton_grouped_gemm_b200.quant.trans_per_block_quant_expand_128x import trans_per_block_quant_expand_128x

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 5e-4


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    _lib.load().b200gemm_set_cta_pair(-1)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("pair", [0, 1])
def test_single_block_known_answer(pair):
    """One expert of 128 tokens, small integers, power-of-two scales: exact."""
    _lib.load().b200gemm_set_cta_pair(pair)
    m = n = t = 128
    x = ((torch.arange(m)[:, None] + torch.arange(t)[None, :]) % 5 - 2).float()
    y = ((torch.arange(n)[:, None] * 2 + torch.arange(t)[None, :]) % 7 - 3).float()
    ref = (x @ y.t()) * 0.5 * 0.25
    out = k_grouped_fp8_block_scaled((x.to(torch.float8_e4m3fn).to(DEV), torch.full((1, 1), 0.5, device=DEV)),
                                     (y.to(torch.float8_e4m3fn).to(DEV), torch.full((1, 1), 0.25, device=DEV)),
                                     torch.tensor([t], device=DEV)).cpu()
    assert out.shape == (1, m, n)
    assert torch.equal(out[0].float(), ref.bfloat16().float())


@pytest.mark.parametrize("pair", [0, 1, -1], ids=["single", "pair", "auto"])
@pytest.mark.parametrize("sizes,k_in,n_out", [
    ([128], 128, 128),
    ([200, 0, 1, 127, 300], 256, 512),
    ([5, 700, 64], 384, 640),          # m_dim = 384: the second CTA of a pair tile hangs over the edge
    ([130] * 9, 512, 256),
])
def test_wgrad_vs_oracle(sizes, k_in, n_out, pair):
    _lib.load().b200gemm_set_cta_pair(pair)
    gen = torch.Generator().manual_seed(k_in + n_out + len(sizes))
    m = sum(sizes)
    a = torch.randn(m, k_in, generator=gen).bfloat16()
    dy = (torch.randn(m, n_out, generator=gen) * 0.1).bfloat16()
    st = torch.tensor(sizes)
    aq, a_s, padded = trans_per_block_quant_expand_128x(a.to(DEV), st.to(DEV))
    gq, g_s, padded2 = trans_per_block_quant_expand_128x(dy.to(DEV), st.to(DEV))
    assert torch.equal(padded, padded2)
    out = k_grouped_fp8_block_scaled((aq, a_s), (gq, g_s), padded).cpu()
    assert out.shape == (len(sizes), k_in, n_out) and out.dtype == torch.bfloat16
    # oracle on the oracle's own quantiser output (bit-identical to the GPU quantiser's, checked elsewhere)
    aq_r, as_r, pad_r = O.trans_quant_expand_ref(a, st)
    gq_r, gs_r, _ = O.trans_quant_expand_ref(dy, st)
    assert torch.equal(aq.cpu().view(torch.uint8), aq_r.view(torch.uint8)) and torch.equal(a_s.cpu(), as_r)
    ref = O.fp8_block_k_grouped_ref(aq_r, as_r, gq_r, gs_r, pad_r)
    assert O.rdiff(out.float(), ref.float()) < TOL
    for g, s in enumerate(sizes):
        if s == 0:
            assert torch.all(out[g] == 0)
    # and close to the unquantised weight gradient (fp8 quantisation noise only)
    full = O.k_grouped_ref(a, dy, st, fp32_accumulate_explicit=True).float()
    assert O.rdiff(out.float(), full) < 0.06
    # the convenience entry point is the same computation, and so is the unbalanced tile order
    assert torch.equal(fp8_wgrad(a.to(DEV), dy.to(DEV), st.to(DEV)).cpu(), out)
    assert torch.equal(k_grouped_fp8_block_scaled((aq, a_s), (gq, g_s), padded, balanced=False).cpu(), out)


def test_rejections():
    lib = _lib.load()
    x = torch.zeros(128, 128, dtype=torch.uint8, device=DEV)
    s = torch.ones(1, 1, device=DEV)
    out = torch.empty(1, 128, 128, dtype=torch.bfloat16, device=DEV)
    sz = torch.tensor([128], device=DEV)
    args = lambda m_expand, m_dim, n_dim: (x.data_ptr(), s.data_ptr(), x.data_ptr(), s.data_ptr(), out.data_ptr(),  # noqa: E731
                                           sz.data_ptr(), 1, 1, m_expand, m_dim, n_dim, None, 0, -1, None)
    assert lib.b200gemm_fp8_k_grouped_block(*args(100, 128, 128)) == -1 and "m_expand" in _lib.last_error()
    assert lib.b200gemm_fp8_k_grouped_block(*args(128, 64, 128)) == -1 and "multiples of 128" in _lib.last_error()


def test_full_size_properties():
    """Benchmark size (G=128, ~663k tokens, 2048 x 768): exact linearity in the scales over the
    whole output, and for EVERY expert a 16 x 16 patch of its gradient against real arithmetic on
    the host (all of the expert's tokens enter every element)."""
    sizes = O.routing_sizes(128, 655360, seed=2026)
    m = int(sizes.sum())
    gen = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randn(m, 2048, device=DEV, generator=gen, dtype=torch.bfloat16)
    dy = torch.randn(m, 768, device=DEV, generator=gen, dtype=torch.bfloat16) * 0.1
    sz = sizes.to(DEV)
    aq, a_s, padded = trans_per_block_quant_expand_128x(a, sz)
    gq, g_s, _ = trans_per_block_quant_expand_128x(dy, sz)
    del a, dy
    c1 = k_grouped_fp8_block_scaled((aq, a_s), (gq, g_s), padded)
    c2 = k_grouped_fp8_block_scaled((aq, a_s), (gq, g_s * 2), padded)
    assert torch.equal(c1 * 2, c2)
    starts = (torch.cumsum(padded, 0) - padded).tolist()
    pl = padded.tolist()
    for g in range(128):
        s, e = int(starts[g]), int(starts[g] + pl[g])
        r0, c0 = (g * 16) % 2048, (g * 48) % 768
        rb, cb = r0 // 128, c0 // 128
        xd = aq[r0:r0 + 16, s:e].float().cpu() * a_s[rb, s // 128:e // 128].cpu().repeat_interleave(128)[None, :]
        yd = gq[c0:c0 + 16, s:e].float().cpu() * g_s[cb, s // 128:e // 128].cpu().repeat_interleave(128)[None, :]
        ref = (xd @ yd.t()).bfloat16()
        assert O.rdiff(c1[g, r0:r0 + 16, c0:c0 + 16].float().cpu(), ref.float()) < TOL, f"expert {g}"
