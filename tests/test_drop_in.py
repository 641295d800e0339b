"""Drop-in proof: code written against the reference's module paths (``from gemm... import``,
``from quant... import``) runs on this package after ``install_as_reference_modules()``.

The CPU part replays the assertions of the reference's own unit test
(tests/test_layout_backend.py:22-59 of the reference) through the installed top-level modules -
with 'b200' where the reference says 'triton', the one documented difference.  The GPU part
calls every operator through its reference import path on a small problem and checks it
against the oracle."""

import sys

import pytest
import torch

import oracle as O
import triton_grouped_gemm_b200 as pkg


@pytest.fixture()
def reference_paths():
    saved = {k: v for k, v in sys.modules.items() if k == "gemm" or k.startswith("gemm.") or k == "quant" or k.startswith("quant.")}
    pkg.install_as_reference_modules(force=True)
    yield
    for k in [k for k in sys.modules if k == "gemm" or k.startswith("gemm.") or k == "quant" or k.startswith("quant.")]:
        del sys.modules[k]
    sys.modules.update(saved)


def test_reference_layout_and_backend_unit_test_through_installed_modules(reference_paths):
    from gemm.backends import GemmBackend, normalize_backend, select_backend
    from gemm.layout import (make_deep_gemm_grouped_layout, make_deep_gemm_psum_layout, make_group_starts,
                             make_grouped_layout, round_up_to_alignment, validate_total_m)

    import gemm

    assert "triton_grouped_gemm_b200" in gemm.__file__
    sizes = torch.tensor([0, 1, 127, 128, 129], dtype=torch.int32)
    assert round_up_to_alignment(sizes, 128).tolist() == [0, 128, 128, 128, 256]
    sizes = torch.tensor([3, 5, 0, 7], dtype=torch.int32)
    assert make_group_starts(sizes, padded=False, block_m=4).tolist() == [0, 3, 8, 8]
    assert make_group_starts(sizes, padded=True, block_m=4).tolist() == [0, 4, 12, 12]
    layout = make_grouped_layout([3, 5, 0, 7], block_m=4)
    assert layout.sizes.tolist() == [3, 5, 0, 7]
    assert layout.padded_sizes.tolist() == [4, 8, 0, 8]
    assert layout.starts.tolist() == [0, 4, 12, 12]
    assert int(layout.total_m.item()) == 15 and int(layout.total_padded_m.item()) == 20
    assert make_deep_gemm_grouped_layout([3, 5], block_m=4).tolist() == [0, 0, 0, -1, 1, 1, 1, 1, 1, -1, -1, -1]
    assert make_deep_gemm_psum_layout([3, 5], block_m=4).tolist() == [3, 9]
    validate_total_m([2, 3, 4], 9)
    with pytest.raises(ValueError, match=r"sum\(size_per_group\)"):
        validate_total_m([2, 3, 4], 10)
    # backends: 'b200' takes the place of 'triton'
    assert normalize_backend("b200") == GemmBackend.B200
    assert normalize_backend("deepgemm") == GemmBackend.DEEP_GEMM
    assert select_backend("b200") == GemmBackend.B200
    with pytest.raises(ValueError, match="Unsupported GEMM backend"):
        normalize_backend("cutlass")
    with pytest.raises(ValueError, match="Unsupported GEMM backend"):
        normalize_backend("triton")
    with pytest.raises(ModuleNotFoundError):
        import gemm.tma  # noqa: F401  (dropped with the Triton backend)


@pytest.mark.gpu
def test_every_operator_through_its_reference_import_path(reference_paths):
    from gemm.BF16.k_grouped_gemm import k_grouped_gemm as k_grouped_gemm_sm80
    from gemm.BF16.k_grouped_gemm_TMA import gmm_dw_reference, k_grouped_gemm
    from gemm.BF16.m_grouped_gemm import m_grouped_gemm as m_grouped_gemm_sm80
    from gemm.BF16.m_grouped_gemm_masked_TMA import m_grouped_gemm_masked
    from gemm.BF16.m_grouped_gemm_TMA import m_grouped_gemm, m_grouped_reference
    from gemm.deep_gemm_ops import m_grouped_fp8_nt_contiguous
    from gemm.FP8.k_grouped_gemm_channel_expert import matmul
    from gemm.FP8.m_grouped_gemm_channel_expert import gmm_fp8_act_per_channel_w_per_expert
    from quant.trans_per_block_quant_expand_128x import trans_per_block_quant_expand_128x, trans_quant

    from triton_grouped_gemm_b200 import _lib

    dev = "cuda"
    a, b, sizes = O.config0_inputs(0)                      # the CPU-reference configuration: G=4, K=512, N=256
    ref = O.m_grouped_ref(a, b, sizes, True, fp32_accumulate_explicit=True)
    for fn in (m_grouped_gemm, m_grouped_gemm_sm80):
        out = fn(a.to(dev), b.to(dev), sizes.to(dev), True)
        assert O.rdiff(out.cpu().float(), ref.float()) <= 2e-3
    # the reference's own torch reference, importable from the same module path, agrees
    assert O.rdiff(m_grouped_reference(a, b, sizes, True).float(), ref.float()) <= 2e-3
    # masked
    g_, e_, k_, n_ = 3, 128, 64, 48
    gen = torch.Generator().manual_seed(1)
    lhs = (torch.randn(g_ * e_, k_, generator=gen) * 0.5).bfloat16()
    rhs = (torch.randn(g_, n_, k_, generator=gen) * 0.5).bfloat16()
    masked = torch.tensor([17, 0, 128])
    out = torch.zeros(g_ * e_, n_, dtype=torch.bfloat16, device=dev)
    assert m_grouped_gemm_masked(lhs.to(dev), rhs.to(dev), out, masked.to(dev), e_) is None
    assert O.rdiff(out.cpu().float(), O.m_grouped_masked_ref(lhs, rhs, torch.zeros(g_ * e_, n_, dtype=torch.bfloat16),
                                                             masked, e_).float()) <= 2e-3
    # K-grouped, both module paths
    ks = torch.tensor([33, 0, 64, 7])
    ka = (torch.randn(int(ks.sum()), 48, generator=gen) * 0.5).bfloat16()
    kb = (torch.randn(int(ks.sum()), 40, generator=gen) * 0.5).bfloat16()
    kref = O.k_grouped_ref(ka, kb, ks)
    for fn in (k_grouped_gemm, k_grouped_gemm_sm80):
        assert O.rdiff(fn(ka.to(dev), kb.to(dev), ks.to(dev)).cpu().float(), kref.float()) <= 2e-3
    assert gmm_dw_reference(ka, kb, ks).shape == kref.shape
    # FP8 row x channel scales, M- and K-grouped
    x = torch.randn(256, 256, generator=gen).bfloat16()
    a8, a_s = O.per_channel_cast_to_fp8(x, torch.float8_e5m2)
    b8 = (torch.randn(2, 256, 256, generator=gen) * 100).clamp(-400, 400).to(torch.float8_e4m3fn)
    b_s = torch.rand(2, 256, generator=gen) * 0.01 + 0.001
    out = gmm_fp8_act_per_channel_w_per_expert(a8.to(dev), a_s.to(dev), b8.to(dev), b_s.reshape(-1).to(dev),
                                               torch.tensor([100, 156], dtype=torch.int32, device=dev), torch.bfloat16)
    assert O.rdiff(out.cpu().float(), O.fp8_rowcol_m_grouped_ref(a8, a_s, b8, b_s, [100, 156], torch.bfloat16).float()) <= 2e-3
    x8 = (torch.randn(128, 384, generator=gen) * 50).to(torch.float8_e4m3fn)
    y8 = (torch.randn(256, 384, generator=gen) * 50).to(torch.float8_e4m3fn)
    xs = (torch.rand(2, 128, generator=gen) * 0.01 + 0.001).t()
    ys = (torch.rand(2, 256, generator=gen) * 0.01 + 0.001).t()
    out = matmul(x8.to(dev), xs.to(dev), y8.to(dev), ys.to(dev), torch.tensor([256, 128], dtype=torch.int32, device=dev),
                 128, 256, 384, 2)
    assert O.rdiff(out.cpu().float(), O.fp8_rowcol_k_grouped_ref(x8, xs, y8, ys, [256, 128], 128, 256, 2).float()) <= 2e-3
    # the quantiser and the DeepGEMM-style wrapper
    xin = torch.randn(300, 256, generator=gen).bfloat16()
    t = torch.tensor([130, 0, 170])
    q, s, pad = trans_per_block_quant_expand_128x(xin.to(dev), t.to(dev))
    q_ref, s_ref, pad_ref = O.trans_quant_expand_ref(xin, t)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s.cpu(), s_ref)
    assert pad.cpu().tolist() == pad_ref.tolist()
    assert callable(trans_quant)
    a8q, a_sq = O.per_token_cast_to_fp8(torch.randn(256, 256, generator=gen).bfloat16())
    wq = [O.per_block_cast_to_fp8((torch.randn(128, 256, generator=gen) * 0.02).bfloat16()) for _ in range(2)]
    b8q, b_sq = torch.stack([w[0] for w in wq]), torch.stack([w[1] for w in wq])
    out = m_grouped_fp8_nt_contiguous((a8q.to(dev), a_sq.to(dev)), (b8q.to(dev), b_sq.to(dev)),
                                      torch.tensor([100, 128], device=dev))
    ref0 = O.fp8_block_m_grouped_ref(a8q[:100], a_sq[:100], b8q[:1], b_sq[:1], [100])
    assert O.rdiff(out[:100].cpu().float(), ref0.float()) <= 2e-3
    assert _lib.device_status() == 0
