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
    # the fixture comes from the reference's torch helper; the operator's clamp of the scale to
    # [1e-12, 3e38] touches no block of it, so both forms of the oracle must reproduce it
    for clamp_scale in (False, True):
        q, s, pad = O.trans_quant_expand_ref(c["x"], c["sizes"], clamp_scale=clamp_scale)
        assert torch.equal(_u8(q), c["q"])
        assert torch.equal(s.view(torch.int32), c["s"].view(torch.int32))
        assert pad.tolist() == c["padded"].tolist()


def test_trans_quant_scale_clamp_of_the_shipped_operator():
    """quant/trans_per_block_quant_expand_128x.py:124-126: scale = clamp(amax / fmax, 1e-12, 3e38).
    An all-zero block: zero bytes (sign kept) and scale float32(1e-12); a block whose amax / 448 is
    below 1e-12 is divided by 1e-12; the torch helper alone gives scale 0 and NaN bytes."""
    x = torch.randn(384, 128).to(torch.bfloat16)
    x[128:256] = 0
    x[130, 5] = -0.0
    x[256:384] = (torch.randn(128, 128) * 1e-11).to(torch.bfloat16)
    sizes = torch.tensor([384])
    q, s, _ = O.trans_quant_expand_ref(x, sizes)
    tiny = torch.tensor(1e-12, dtype=torch.float32)
    assert s[0, 1] == tiny and s[0, 2] == tiny and s[0, 0] > 1e-3
    qb = _u8(q)
    assert set(qb[:, 128:256].unique().tolist()) <= {0x00, 0x80}
    assert qb[5, 130] == 0x80
    expect = (x[256:384].float() / tiny).clamp(-448, 448).to(torch.float8_e4m3fn).t()
    assert torch.equal(qb[:, 256:384], _u8(expect))
    q0, s0, _ = O.trans_quant_expand_ref(x, sizes, clamp_scale=False)
    assert s0[0, 1] == 0 and bool((_u8(q0)[:, 128:256] == 0xFF).all())
    assert torch.equal(_u8(q0)[:, :128], qb[:, :128]) and s0[0, 0] == s[0, 0]


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


# ---------------------------------------------------------------- FP8 row x channel GEMMs
# fp8_rowcol.pt holds what the reference's own Triton kernels computed on a B200
# (tests/golden/make_golden_gpu.py); the inputs are rebuilt here from the seed and must hash to
# what the kernels were given.

def _rowcol_casts():
    return {"per_channel_cast_to_fp8": O.per_channel_cast_to_fp8, "per_expert_cast_to_fp8": O.per_expert_cast_to_fp8}


def _rowcol_cases():
    import sys

    from conftest import GOLDEN

    if str(GOLDEN) not in sys.path:
        sys.path.insert(0, str(GOLDEN))
    import fp8_rowcol_cases as C

    return C


@pytest.mark.parametrize("name", ["one_tile_e4e4", "ragged_e5e4_fp16", "ragged_e4e4_ktail", "test_family_e5e4"])
def test_fp8_rowcol_m_grouped_oracle_vs_reference_kernel(golden_dir, name):
    C = _rowcol_cases()
    e = _load(golden_dir, "fp8_rowcol.pt")["m_grouped"][name]
    assert "out" in e, e.get("error")
    inp = C.m_case_inputs(name, _rowcol_casts())
    assert C.input_hashes(inp) == e["inputs_sha256"]
    ref = O.fp8_rowcol_m_grouped_ref(inp["a8"], inp["a_scale"], inp["b8"], inp["b_scale"], inp["sizes"], inp["dtype_out"])
    assert ref.dtype == e["out"].dtype and ref.shape == e["out"].shape
    # same products, fp32 accumulation in a different order, one rounding: measured 0 .. 7e-10
    assert O.rdiff(ref.float(), e["out"].float()) < 5e-4


@pytest.mark.parametrize("name", ["one_tile_e4e4", "ragged_e4e4", "ragged_e5e4"])
def test_fp8_rowcol_k_grouped_oracle_vs_reference_kernel(golden_dir, name):
    C = _rowcol_cases()
    e = _load(golden_dir, "fp8_rowcol.pt")["k_grouped"][name]
    assert "out" in e, e.get("error")
    inp = C.k_case_inputs(name, _rowcol_casts())
    assert C.input_hashes(inp) == e["inputs_sha256"]
    g = inp["tokens"].numel()
    assert inp["x_scale"].shape == (inp["m"], g) and (g == 1 or inp["x_scale"].stride() == (1, inp["m"]))  # group-major
    ref = O.fp8_rowcol_k_grouped_ref(inp["x8"], inp["x_scale"], inp["y8"], inp["y_scale"], inp["tokens"], inp["m"],
                                     inp["n"], g)
    assert ref.shape == e["out"].shape
    assert O.rdiff(ref.float(), e["out"].float()) < 5e-4  # measured 0 .. 6e-8
    for i, t in enumerate(inp["tokens"].tolist()):
        if t == 0:
            assert bool((e["out"][i] == 0).all())
