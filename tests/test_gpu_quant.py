"""GPU quantisers against the CPU oracle and the reference-generated fixtures: bytes and
scales must be identical (compared as uint8 / int32 bit patterns)."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.quant.per_block_cast import per_block_cast_to_fp8, per_token_cast_to_fp8
from triton_grouped_gemm_b200.quant.trans_per_block_quant_expand_128x import trans_per_block_quant_expand_128x

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _u8(t):
    return t.contiguous().view(torch.uint8).cpu()


def _bits(t):
    return t.contiguous().view(torch.int32).cpu()


def _assert_same(q, s, q_ref, s_ref):
    dq = (_u8(q) != _u8(q_ref)).sum().item()
    ds = (_bits(s) != _bits(s_ref)).sum().item()
    assert dq == 0 and ds == 0, f"{dq} byte mismatches, {ds} scale mismatches"
    assert _lib.device_status() == 0


def test_per_token_golden(golden_dir):
    c = torch.load(golden_dir / "casts.pt", weights_only=False)["per_token"]
    q, s = per_token_cast_to_fp8(c["x"].to(DEV))
    assert torch.equal(_u8(q), c["q"]) and torch.equal(_bits(s), c["s"].view(torch.int32))


def test_per_block_golden(golden_dir):
    c = torch.load(golden_dir / "casts.pt", weights_only=False)["per_block"]
    q, s = per_block_cast_to_fp8(c["x"].to(DEV))
    assert torch.equal(_u8(q), c["q"]) and torch.equal(_bits(s), c["s"].view(torch.int32))


@pytest.mark.parametrize("name", ["equal", "ragged"])
def test_trans_quant_golden(golden_dir, name):
    c = torch.load(golden_dir / "trans_quant.pt", weights_only=False)[name]
    q, s, pad = trans_per_block_quant_expand_128x(c["x"].to(DEV), c["sizes"].to(DEV))
    assert torch.equal(_u8(q), c["q"]) and torch.equal(_bits(s), c["s"].view(torch.int32))
    assert pad.cpu().tolist() == c["padded"].tolist()


@pytest.mark.parametrize("rows,k,scale,dtype", [
    (1, 128, 1.0, torch.bfloat16), (37, 384, 1.0, torch.bfloat16), (1000, 4096, 1.0, torch.bfloat16),
    (513, 2048, 0.02, torch.bfloat16), (64, 256, 30.0, torch.float16), (3, 128, 1e-6, torch.bfloat16),
])
def test_per_token_vs_oracle(rows, k, scale, dtype):
    gen = torch.Generator().manual_seed(rows * 7 + k)
    x = (torch.randn(rows, k, generator=gen) * scale).to(dtype)
    x[0, :5] = 0
    q_ref, s_ref = O.per_token_cast_to_fp8(x)
    q, s = per_token_cast_to_fp8(x.to(DEV))
    _assert_same(q, s, q_ref, s_ref)


@pytest.mark.parametrize("batch,rows,cols", [(None, 128, 128), (None, 200, 300), (3, 256, 384), (2, 100, 72), (1, 1, 8)])
def test_per_block_vs_oracle(batch, rows, cols):
    gen = torch.Generator().manual_seed(rows + cols)
    shape = (rows, cols) if batch is None else (batch, rows, cols)
    x = (torch.randn(*shape, generator=gen) * 0.02).to(torch.bfloat16)
    q, s = per_block_cast_to_fp8(x.to(DEV))
    if batch is None:
        q_ref, s_ref = O.per_block_cast_to_fp8(x)
    else:
        pairs = [O.per_block_cast_to_fp8(x[i]) for i in range(batch)]
        q_ref = torch.stack([p[0] for p in pairs])
        s_ref = torch.stack([p[1] for p in pairs])
    _assert_same(q, s, q_ref, s_ref)


@pytest.mark.parametrize("sizes,n", [
    ([128], 128), ([1], 128), ([127, 129], 256), ([0, 5, 0, 300, 128], 384), ([256] * 8, 512),
    ([77, 0, 0, 1, 640, 3], 128),
])
def test_trans_quant_vs_oracle(sizes, n):
    gen = torch.Generator().manual_seed(sum(sizes) + n)
    x = torch.randn(sum(sizes), n, generator=gen).to(torch.bfloat16)
    t = torch.tensor(sizes)
    q_ref, s_ref, pad_ref = O.trans_quant_expand_ref(x, t)
    for st in (t.to(torch.int64), t.to(torch.int32)):
        q, s, pad = trans_per_block_quant_expand_128x(x.to(DEV), st.to(DEV))
        assert q.shape == q_ref.shape and s.shape == s_ref.shape
        _assert_same(q, s, q_ref, s_ref)
        assert pad.cpu().tolist() == pad_ref.tolist()


def test_trans_quant_large_random_is_bit_exact():
    """32M elements with block magnitudes spread over 60 binades: every byte must match the host's
    fp32 division + clamp + cast.  The kernel brackets each quotient between two directed-rounding
    products and only divides where the bracket straddles an e4m3 rounding boundary; at this size
    about a hundred elements take that route."""
    gen = torch.Generator().manual_seed(77)
    rows, n = 16384, 2048
    x = torch.randn(rows, n, generator=gen)
    mag = torch.exp2(torch.randint(-30, 30, (rows // 128, 1, n // 128, 1), generator=gen).float())
    x = (x.view(rows // 128, 128, n // 128, 128) * mag).view(rows, n).bfloat16()
    t = torch.tensor([1024, 0, 777, 2295 + 12288])
    q_ref, s_ref, _ = O.trans_quant_expand_ref(x, t)
    q, s, _ = trans_per_block_quant_expand_128x(x.to(DEV), t.to(DEV))
    _assert_same(q, s, q_ref, s_ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_trans_quant_extreme_blocks_and_signed_zeros(dtype):
    """Blocks whose scale is tiny, huge or subnormal, exact e4m3 ties, and negative zeros."""
    gen = torch.Generator().manual_seed(5)
    rows, n = 1024, 512
    x = torch.randn(rows, n, generator=gen)
    lo, hi = (-125, 121) if dtype == torch.bfloat16 else (-22, 13)
    mag = torch.exp2(torch.randint(lo, hi, (rows // 128, 1, n // 128, 1), generator=gen).float())
    x = (x.view(rows // 128, 128, n // 128, 128) * mag).view(rows, n).to(dtype)
    # one block with scale exactly 1 and values on e4m3 rounding ties
    x[:128, :128] = torch.tensor([1.0625, -1.1875, 0.0009765625, 17.0, -0.0, 0.0, 448.0, -26.0]).repeat(128, 16).to(dtype)
    x[128:256, 128:256][::2] = -0.0
    assert torch.isfinite(x.float()).all()
    t = torch.tensor([300, 724])
    q_ref, s_ref, _ = O.trans_quant_expand_ref(x, t)
    q, s, _ = trans_per_block_quant_expand_128x(x.to(DEV), t.to(DEV))
    _assert_same(q, s, q_ref, s_ref)


def test_trans_quant_all_zero_and_tiny_blocks_follow_the_operators_scale_clamp():
    """The reference's shipped operator clamps the block scale to [1e-12, 3e38]
    (quant/trans_per_block_quant_expand_128x.py:124-126): an all-zero block gives zero bytes
    and scale 1e-12 (not the torch helper's scale 0 and NaN bytes), and nothing downstream sees
    a NaN."""
    x = torch.randn(384, 128).to(torch.bfloat16)
    x[128:256] = 0  # second 128x128 block of the only expert is all zero
    x[130, 5] = -0.0
    x[256:384] = (torch.randn(128, 128) * 1e-11).to(torch.bfloat16)  # amax / 448 below the clamp
    t = torch.tensor([384])
    q_ref, s_ref, _ = O.trans_quant_expand_ref(x, t)
    q, s, _ = trans_per_block_quant_expand_128x(x.to(DEV), t.to(DEV))
    _assert_same(q, s, q_ref, s_ref)
    assert float(s[0, 1]) == float(torch.tensor(1e-12, dtype=torch.float32))
    assert not torch.isnan(q.float()).any()


def test_full_size_linearity_property():
    """At benchmark size the oracle is too slow; use a property instead: scaling the input by a
    power of two leaves the bytes unchanged and scales the scales by exactly that factor."""
    rows, k = 65536, 4096
    x = torch.randn(rows, k, device=DEV, dtype=torch.bfloat16)
    q1, s1 = per_token_cast_to_fp8(x)
    q2, s2 = per_token_cast_to_fp8(x * 4)
    assert torch.equal(q1.view(torch.uint8), q2.view(torch.uint8))
    assert torch.equal(s1 * 4, s2)
    # and a slice of it agrees with the oracle
    q_ref, s_ref = O.per_token_cast_to_fp8(x[:512].cpu())
    _assert_same(q1[:512], s1[:512], q_ref, s_ref)
