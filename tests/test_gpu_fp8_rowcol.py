"""FP8 grouped GEMMs with per-row x per-channel scales against the CPU oracle (dequantised
fp32 reference of the same fp8 bytes) and against outputs of the reference's own Triton kernels
(tests/golden/fp8_rowcol.pt, made on a B200 by tests/golden/make_golden_gpu.py).  Tolerance
rdiff <= 2e-3; only accumulation order and the final rounding differ, so 5e-4 is asserted."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.gemm.FP8.k_grouped_gemm_channel_expert import matmul
from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_channel_expert import gmm_fp8_act_per_channel_w_per_expert

pytestmark = pytest.mark.gpu
DEV = "cuda"
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    _lib.load().b200gemm_set_block_n(0)
    _lib.load().b200gemm_set_cta_pair(-1)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("block_n", [0, 64, 128, 256])
@pytest.mark.parametrize("dt_a,dt_b", [(E4, E4), (E5, E4)])
@pytest.mark.parametrize("sizes,n,k,dtype_out", [
    ([128], 256, 128, torch.bfloat16),
    ([125, 0, 509, 3], 384, 640, torch.float16),
    ([300, 77], 264, 272, torch.bfloat16),     # n and k tails
])
def test_m_grouped_rowcol(sizes, n, k, dtype_out, dt_a, dt_b, block_n):
    gen = torch.Generator().manual_seed(n + k + len(sizes))
    m, g = sum(sizes), len(sizes)
    x = torch.randn(m + 5, (k + 127) // 128 * 128, generator=gen).bfloat16()
    w = torch.randn(g, 128, 128, generator=gen).bfloat16()
    a8, a_s = O.per_channel_cast_to_fp8(x, dt_a)
    a8 = a8[:, :k].contiguous()
    b8 = (torch.randn(g, n, k, generator=gen) * 100).clamp(-400, 400).to(dt_b)
    b_s = torch.rand(g, n, generator=gen) * 0.01 + 0.001
    del w
    ref = O.fp8_rowcol_m_grouped_ref(a8[:m], a_s[:m], b8, b_s, sizes, dtype_out)
    _lib.load().b200gemm_set_block_n(block_n)
    out = gmm_fp8_act_per_channel_w_per_expert(a8.to(DEV), a_s.to(DEV), b8.to(DEV), b_s.reshape(-1).to(DEV),
                                               torch.tensor(sizes, dtype=torch.int32, device=DEV), dtype_out).cpu()
    assert out.dtype == dtype_out and out.shape == (m + 5, n)
    assert O.rdiff(out[:m].float(), ref.float()) < 5e-4


def test_m_grouped_rowcol_pair_kernel():
    sizes, n, k = [300, 0, 700, 130], 512, 384
    gen = torch.Generator().manual_seed(21)
    m, g = sum(sizes), len(sizes)
    x = torch.randn(m, k, generator=gen).bfloat16()
    a8, a_s = O.per_channel_cast_to_fp8(x, E5)
    b8 = (torch.randn(g, n, k, generator=gen) * 100).clamp(-400, 400).to(E4)
    b_s = torch.rand(g, n, generator=gen) * 0.01 + 0.001
    ref = O.fp8_rowcol_m_grouped_ref(a8, a_s, b8, b_s, sizes, torch.bfloat16)
    _lib.load().b200gemm_set_cta_pair(1)
    out = gmm_fp8_act_per_channel_w_per_expert(a8.to(DEV), a_s.to(DEV), b8.to(DEV), b_s.reshape(-1).to(DEV),
                                               torch.tensor(sizes, dtype=torch.int32, device=DEV), torch.bfloat16).cpu()
    assert O.rdiff(out.float(), ref.float()) < 5e-4


def test_m_grouped_rowcol_reference_test_shape_family():
    """Scaled-down version of the reference's own test (tests/test_FP8/
    test_m_grouped_gemm_channel_expert.py:104-126): ragged experts, e5m2 activations x e4m3
    weights, per-expert weight scale expanded to [G, N]."""
    bias = 3
    tokens = [512 - bias, 1024 - 512 + bias, 128 - bias, 1024 - 128 + bias] * 2
    n, k = 768, 640
    gen = torch.Generator().manual_seed(0)
    m, g = sum(tokens), len(tokens)
    x = torch.randn(m, k, generator=gen).bfloat16()
    w = torch.randn(g, n, k, generator=gen).bfloat16()
    a8, a_s = O.per_channel_cast_to_fp8(x, E5)
    b8, b_s = O.per_expert_cast_to_fp8(w, E4)
    b_s_full = b_s.view(-1, 1).repeat(1, n)
    ref = O.fp8_rowcol_m_grouped_ref(a8, a_s, b8, b_s_full, tokens, torch.bfloat16)
    out = gmm_fp8_act_per_channel_w_per_expert(a8.to(DEV), a_s.to(DEV), b8.to(DEV), b_s_full.to(DEV),
                                               torch.tensor(tokens, dtype=torch.int32, device=DEV),
                                               dtype_out=torch.bfloat16).cpu()
    assert O.rdiff(out.float(), ref.float()) < 5e-4
    # and the quantised product is close to the unquantised one, as the reference's test prints
    full = O.m_grouped_ref(x, w, tokens, True).float()
    assert (out.float() - full).abs().max() / full.abs().max() < 0.1


@pytest.mark.parametrize("pair", [-1, 1, 0], ids=["auto", "pair", "single"])
@pytest.mark.parametrize("dt_a,dt_b", [(E4, E4), (E5, E4)])
@pytest.mark.parametrize("tokens,m,n", [([128], 128, 256), ([256, 0, 128, 512], 256, 384), ([128, 128], 136, 72),
                                        ([1024, 128, 0, 384, 2048], 512, 768)])
def test_k_grouped_rowcol(tokens, m, n, dt_a, dt_b, pair):
    _lib.load().b200gemm_set_cta_pair(pair)
    gen = torch.Generator().manual_seed(m + n + len(tokens))
    g, k_tot = len(tokens), sum(tokens)
    x8 = (torch.randn(m, k_tot, generator=gen) * 50).to(dt_a)
    y8 = (torch.randn(n, k_tot, generator=gen) * 50).to(dt_b)
    # logical [M, G] with group-major memory, as the reference's data generator builds it
    xs = (torch.rand(g, m, generator=gen) * 0.01 + 0.001).t()
    ys = (torch.rand(g, n, generator=gen) * 0.01 + 0.001).t()
    assert xs.stride() == (1, m) or g == 1
    ref = O.fp8_rowcol_k_grouped_ref(x8, xs, y8, ys, tokens, m, n, g)
    out = matmul(x8.to(DEV), xs.to(DEV), y8.to(DEV), ys.to(DEV), torch.tensor(tokens, dtype=torch.int32, device=DEV),
                 m, n, k_tot, g, 1 if dt_a == E4 else 2, 1 if dt_b == E4 else 2).cpu()
    assert out.shape == (g, m, n) and out.dtype == torch.bfloat16
    assert O.rdiff(out.float(), ref.float()) < 5e-4
    for i, t in enumerate(tokens):
        if t == 0:
            assert torch.all(out[i] == 0)


# ---------------------------------------------------------------- against the reference's kernels

def _rowcol_cases():
    import sys

    from conftest import GOLDEN

    if str(GOLDEN) not in sys.path:
        sys.path.insert(0, str(GOLDEN))
    import fp8_rowcol_cases as C

    return C, {"per_channel_cast_to_fp8": O.per_channel_cast_to_fp8, "per_expert_cast_to_fp8": O.per_expert_cast_to_fp8}


@pytest.mark.parametrize("pair", [-1, 0], ids=["auto", "single"])
@pytest.mark.parametrize("name", ["one_tile_e4e4", "ragged_e5e4_fp16", "ragged_e4e4_ktail", "test_family_e5e4"])
def test_m_grouped_rowcol_vs_reference_kernel_output(golden_dir, name, pair):
    C, casts = _rowcol_cases()
    e = torch.load(golden_dir / "fp8_rowcol.pt", weights_only=False)["m_grouped"][name]
    inp = C.m_case_inputs(name, casts)
    assert C.input_hashes(inp) == e["inputs_sha256"]
    _lib.load().b200gemm_set_cta_pair(pair)
    out = gmm_fp8_act_per_channel_w_per_expert(inp["a8"].to(DEV), inp["a_scale"].to(DEV), inp["b8"].to(DEV),
                                               inp["b_scale"].reshape(-1).to(DEV), inp["sizes"].to(DEV),
                                               inp["dtype_out"]).cpu()
    assert out.dtype == e["out"].dtype and out.shape == e["out"].shape
    assert O.rdiff(out.float(), e["out"].float()) < 5e-4


@pytest.mark.parametrize("pair", [-1, 0], ids=["auto", "single"])
@pytest.mark.parametrize("name", ["one_tile_e4e4", "ragged_e4e4", "ragged_e5e4"])
def test_k_grouped_rowcol_vs_reference_kernel_output(golden_dir, name, pair):
    C, casts = _rowcol_cases()
    e = torch.load(golden_dir / "fp8_rowcol.pt", weights_only=False)["k_grouped"][name]
    inp = C.k_case_inputs(name, casts)
    assert C.input_hashes(inp) == e["inputs_sha256"]
    _lib.load().b200gemm_set_cta_pair(pair)
    g, k_tot = inp["tokens"].numel(), int(inp["tokens"].sum())
    xs = inp["x_scale"].t().contiguous().to(DEV).t()   # group-major memory, logical [M, G]
    ys = inp["y_scale"].t().contiguous().to(DEV).t()
    out = matmul(inp["x8"].to(DEV), xs, inp["y8"].to(DEV), ys, inp["tokens"].to(DEV), inp["m"], inp["n"], k_tot, g,
                 inp["dtype_a"], inp["dtype_b"]).cpu()
    assert out.shape == e["out"].shape and out.dtype == e["out"].dtype
    assert O.rdiff(out.float(), e["out"].float()) < 5e-4


def test_m_grouped_rowcol_sizes_past_m_rows_are_cut_off_and_flagged():
    """sum(sizes) > m_rows: nothing at or past row m_rows of C is written (C is a prefix of a larger
    buffer of this test), a_scale is not indexed there, status bit 0x10 is raised."""
    sizes_bad, m_rows, n, k = [200, 300, 128], 400, 256, 256
    gen = torch.Generator().manual_seed(9)
    a8, a_s = O.per_channel_cast_to_fp8(torch.randn(m_rows, k, generator=gen).bfloat16(), E4)
    b8 = (torch.randn(3, n, k, generator=gen) * 100).clamp(-400, 400).to(E4)
    b_s = torch.rand(3, n, generator=gen) * 0.01 + 0.001
    lib = _lib.load()
    c_big = torch.full((m_rows + 256, n), 5.0, device=DEV, dtype=torch.bfloat16)
    a_d, as_d, b_d, bs_d = a8.to(DEV), a_s.reshape(-1).to(DEV), b8.to(DEV), b_s.reshape(-1).to(DEV)
    sz = torch.tensor(sizes_bad, dtype=torch.int32, device=DEV)
    rc = lib.b200gemm_fp8_m_grouped_rowcol(a_d.data_ptr(), as_d.data_ptr(), b_d.data_ptr(), bs_d.data_ptr(),
                                           c_big.data_ptr(), sz.data_ptr(), 0, 3, m_rows, n, k, 0, 0, 0, -1,
                                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    assert _lib.device_status() == 0x10
    out = c_big.cpu()
    assert torch.all(out[m_rows:] == 5.0)
    ref = O.fp8_rowcol_m_grouped_ref(a8, a_s, b8, b_s, [200, 200, 0], torch.bfloat16)
    assert O.rdiff(out[:m_rows].float(), ref.float()) < 5e-4
