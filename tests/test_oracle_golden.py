"""The CPU oracle against fixtures produced by the reference's own torch code
(tests/golden/make_golden.py).  Integer / byte results must be identical; 16-bit GEMM
outputs may differ only by fp32 accumulation order."""

import hashlib

import pytest
import torch

import oracle as O


def _load(golden_dir, name):
    return torch.load(golden_dir / name, weights_only=False)


def _u8(t):
    return t.contiguous().view(torch.uint8)


def _sha(t):
    return hashlib.sha256(_u8(t).numpy().tobytes()).hexdigest()


def test_layouts(golden_dir):
    for case in _load(golden_dir, "layout.pt").values():
        s, bm = case["sizes"], case["block_m"]
        assert O.layout_round_up(s, bm) == case["round_up"]
        assert O.layout_group_starts(s, False, bm) == case["starts"]
        assert O.layout_group_starts(s, True, bm) == case["starts_padded"]
        assert O.layout_grouped(s, bm) == case["grouped_layout"]
        assert O.layout_psum(s, bm) == case["psum"]
        assert O.layout_group_starts(s, True, bm) == case["gl_starts"]
        assert O.layout_round_up(s, bm) == case["gl_padded"]
        assert sum(s) == case["total_m"] and sum(O.layout_round_up(s, bm)) == case["total_padded_m"]


def test_layout_literals_of_reference_unit_test():
    # tests/test_layout_backend.py:22-52 of the reference
    assert O.layout_round_up([0, 1, 127, 128, 129], 128) == [0, 128, 128, 128, 256]
    assert O.layout_group_starts([3, 5, 0, 7], False, 4) == [0, 3, 8, 8]
    assert O.layout_group_starts([3, 5, 0, 7], True, 4) == [0, 4, 12, 12]
    assert O.layout_grouped([3, 5], 4) == [0, 0, 0, -1, 1, 1, 1, 1, 1, -1, -1, -1]
    assert O.layout_psum([3, 5], 4) == [3, 9]


def test_m_grouped(golden_dir):
    g = _load(golden_dir, "m_grouped.pt")
    a, b, sizes = O.config0_inputs(0)
    c0 = g["config0"]
    assert torch.equal(sizes, c0["sizes"]) and _sha(a) == c0["a_sha"] and _sha(b) == c0["b_sha"]
    for explicit in (False, True):
        out = O.m_grouped_ref(a, b, sizes, True, fp32_accumulate_explicit=explicit)
        assert out.shape == c0["out"].shape
        assert O.rdiff(out, c0["out"]) < 2e-4  # accumulation order only (bf16 ulp flips)
    for name, tb in (("small_nt", True), ("small_nn", False), ("small_nt_fp16", True)):
        c = g[name]
        for explicit in (False, True):
            out = O.m_grouped_ref(c["a"], c["b"], c["sizes"], tb, fp32_accumulate_explicit=explicit)
            assert out.dtype == c["out"].dtype
            assert O.rdiff(out, c["out"]) < 2e-4


def test_masked(golden_dir):
    c = _load(golden_dir, "masked.pt")
    e = c["expected_m"]
    sentinel = torch.full_like(c["full"], 7.0)
    out = O.m_grouped_masked_ref(c["lhs"], c["rhs"], sentinel, c["masked_m"], e)
    for g, m in enumerate(c["masked_m"].tolist()):
        assert O.rdiff(out[g * e:g * e + m], c["full"][g * e:g * e + m]) < 2e-4
        assert torch.all(out[g * e + m:(g + 1) * e] == 7.0)  # untouched rows


def test_k_grouped(golden_dir):
    c = _load(golden_dir, "k_grouped.pt")
    for explicit in (False, True):
        out = O.k_grouped_ref(c["a"], c["b"], c["sizes"], fp32_accumulate_explicit=explicit)
        assert out.shape == c["out"].shape
        assert O.rdiff(out, c["out"]) < 2e-4
    assert torch.all(out[1] == 0)


@pytest.mark.parametrize("name", ["per_token", "per_block", "per_channel_e4m3", "per_channel_e5m2",
                                  "per_expert_e4m3", "per_expert_e5m2"])
def test_casts_bit_exact(golden_dir, name):
    c = _load(golden_dir, "casts.pt")[name]
    if name == "per_token":
        q, s = O.per_token_cast_to_fp8(c["x"])
    elif name == "per_block":
        q, s = O.per_block_cast_to_fp8(c["x"])
    elif name.startswith("per_channel"):
        q, s = O.per_channel_cast_to_fp8(c["x"], torch.float8_e4m3fn if "e4m3" in name else torch.float8_e5m2)
    else:
        q, s = O.per_expert_cast_to_fp8(c["x"], torch.float8_e4m3fn if "e4m3" in name else torch.float8_e5m2)
    assert torch.equal(_u8(q), c["q"])
    assert torch.equal(s.view(torch.int32), c["s"].view(torch.int32))


@pytest.mark.parametrize("name", ["equal", "ragged"])
def test_trans_quant_bit_exact(golden_dir, name):
    c = _load(golden_dir, "trans_quant.pt")[name]
    q, s, pad = O.trans_quant_expand_ref(c["x"], c["sizes"])
    assert torch.equal(_u8(q), c["q"])
    assert torch.equal(s.view(torch.int32), c["s"].view(torch.int32))
    assert pad.tolist() == c["padded"].tolist()


def test_dequant_roundtrip_is_close():
    torch.manual_seed(0)
    x = torch.randn(16, 256).to(torch.bfloat16)
    q, s = O.per_token_cast_to_fp8(x)
    assert O.rdiff(O.dequant_1x128(q, s), x.float()) < 0.04
    w = (torch.randn(256, 128) * 0.02).to(torch.bfloat16)
    q, s = O.per_block_cast_to_fp8(w)
    assert O.rdiff(O.dequant_128x128(q, s), w.float()) < 0.04


def test_routing_sizes_deterministic():
    s = O.routing_sizes(128, 655360, seed=2026)
    assert s.numel() == 128 and int((s % 128).abs().sum()) == 0
    assert 655360 <= int(s.sum()) <= 655360 + 128 * 128
    assert torch.equal(s, O.routing_sizes(128, 655360, seed=2026))
