"""Layout / backend helpers: the reference's own unit test (tests/test_layout_backend.py:22-59)
restated against this package, with 'triton' replaced by 'b200', plus the golden fixtures."""

import pytest
import torch

from triton_grouped_gemm_b200.gemm.backends import GemmBackend, normalize_backend, select_backend
from triton_grouped_gemm_b200.gemm.layout import (
    as_group_sizes,
    device_group_metadata,
    make_deep_gemm_grouped_layout,
    make_deep_gemm_psum_layout,
    make_group_starts,
    make_grouped_layout,
    round_up_to_alignment,
    validate_total_m,
)
import oracle as O


def test_round_up_to_alignment():
    sizes = torch.tensor([0, 1, 127, 128, 129], dtype=torch.int32)
    assert round_up_to_alignment(sizes, 128).tolist() == [0, 128, 128, 128, 256]
    with pytest.raises(ValueError, match="alignment must be positive"):
        round_up_to_alignment(sizes, 0)


def test_make_group_starts_logical_and_padded():
    sizes = torch.tensor([3, 5, 0, 7], dtype=torch.int32)
    assert make_group_starts(sizes, padded=False, block_m=4).tolist() == [0, 3, 8, 8]
    assert make_group_starts(sizes, padded=True, block_m=4).tolist() == [0, 4, 12, 12]


def test_make_grouped_layout_summary():
    layout = make_grouped_layout([3, 5, 0, 7], block_m=4)
    assert layout.sizes.tolist() == [3, 5, 0, 7]
    assert layout.padded_sizes.tolist() == [4, 8, 0, 8]
    assert layout.starts.tolist() == [0, 4, 12, 12]
    assert int(layout.total_m.item()) == 15
    assert int(layout.total_padded_m.item()) == 20


def test_make_deep_gemm_grouped_layout():
    assert make_deep_gemm_grouped_layout([3, 5], block_m=4).tolist() == [0, 0, 0, -1, 1, 1, 1, 1, 1, -1, -1, -1]


def test_make_deep_gemm_psum_layout():
    assert make_deep_gemm_psum_layout([3, 5], block_m=4).tolist() == [3, 9]


def test_validate_total_m():
    validate_total_m([2, 3, 4], 9)
    with pytest.raises(ValueError, match=r"sum\(size_per_group\)"):
        validate_total_m([2, 3, 4], 10)


def test_size_validation_errors():
    with pytest.raises(ValueError, match="must be 1D"):
        as_group_sizes(torch.zeros(2, 2, dtype=torch.int32))
    with pytest.raises(ValueError, match="at least one group"):
        as_group_sizes([])
    with pytest.raises(ValueError, match="negative"):
        as_group_sizes([1, -1])


def test_backend_normalization_and_b200_selection():
    assert normalize_backend("b200") == GemmBackend.B200
    assert normalize_backend("deepgemm") == GemmBackend.DEEP_GEMM
    assert normalize_backend("deep-gemm") == GemmBackend.DEEP_GEMM
    assert select_backend("b200") == GemmBackend.B200
    assert select_backend("auto") == GemmBackend.B200
    assert select_backend() == GemmBackend.B200
    with pytest.raises(ValueError, match="Unsupported GEMM backend"):
        normalize_backend("cutlass")
    with pytest.raises(ValueError, match="Unsupported GEMM backend"):
        normalize_backend("triton")  # replaced by 'b200'


def test_layouts_match_golden(golden_dir):
    for case in torch.load(golden_dir / "layout.pt", weights_only=False).values():
        s, bm = case["sizes"], case["block_m"]
        t = torch.tensor(s, dtype=torch.int32)
        assert round_up_to_alignment(t, bm).tolist() == case["round_up"]
        assert make_group_starts(t, padded=False, block_m=bm).tolist() == case["starts"]
        assert make_group_starts(t, padded=True, block_m=bm).tolist() == case["starts_padded"]
        assert make_deep_gemm_grouped_layout(s, block_m=bm).tolist() == case["grouped_layout"]
        assert make_deep_gemm_psum_layout(s, block_m=bm).tolist() == case["psum"]
        gl = make_grouped_layout(s, block_m=bm)
        assert gl.starts.tolist() == case["gl_starts"] and gl.padded_sizes.tolist() == case["gl_padded"]


def test_device_group_metadata_matches_oracle():
    sizes = [130, 0, 1, 128, 257]
    ps, pe, gs, ge, idx, mpad = device_group_metadata(torch.tensor(sizes), 128)
    ops, ope, ogs, oge, oidx, ompad = O.layout_m_grouped_metadata(sizes, 128)
    assert ps.tolist() == ops and pe.tolist() == ope and gs.tolist() == ogs and ge.tolist() == oge
    assert idx[: len(oidx)].tolist() == oidx and int(mpad) == ompad
    assert idx.numel() == sum(sizes) // 128 + len(sizes)
