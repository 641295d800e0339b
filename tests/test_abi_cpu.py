"""The C-ABI library without a GPU: it loads, exports every symbol the header declares,
and rejects bad arguments on the host with an error code and a message."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

from triton_grouped_gemm_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def _declared_functions():
    text = (ROOT / "include" / "b200gemm.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = _lib.load()
    names = _declared_functions()
    assert len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/b200gemm.h but not exported"
    assert set(names) == set(_lib.EXPORTED_SYMBOLS), "ctypes signature table and header disagree"


def test_version_and_last_error():
    lib = _lib.load()
    assert lib.b200gemm_version() >= 100
    assert isinstance(_lib.last_error(), str)


def test_host_side_rejections_need_no_gpu():
    lib = _lib.load()
    # k not a multiple of 8 -> invalid argument, before any device work
    rc = lib.b200gemm_m_grouped(16, 16, 16, 16, 0, 1, 128, 64, 12, 1, 0, -1, None)
    assert rc == -1 and "16-byte alignment" in _lib.last_error()
    rc = lib.b200gemm_m_grouped(16, 16, 16, 16, 0, 1, 128, 64, 64, 1, 7, -1, None)
    assert rc == -1 and "dtype" in _lib.last_error()
    rc = lib.b200gemm_m_grouped(8, 16, 16, 16, 0, 1, 128, 64, 64, 1, 0, -1, None)
    assert rc == -1 and "aligned" in _lib.last_error()
    rc = lib.b200quant_act_1x128(16, 16, 16, 4, 100, 0, None)
    assert rc == -1 and "multiple of 128" in _lib.last_error()
    rc = lib.b200quant_trans_expand_128x(16, 16, 0, 2, 16, 16, None, 256, 100, 512, 0, None)
    assert rc == -1 and "multiple of 128" in _lib.last_error()
    rc = lib.b200gemm_set_block_n(100)
    assert rc == -1
    assert lib.b200gemm_set_block_n(0) == 0
    # empty problems are accepted without touching a device
    assert lib.b200gemm_m_grouped(None, None, None, None, 0, 0, 0, 64, 64, 1, 0, -1, None) == 0


def test_python_layer_refuses_cpu_tensors():
    from triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_TMA import _m_grouped_gemm_launch
    from triton_grouped_gemm_b200.quant.per_block_cast import per_token_cast_to_fp8

    a = torch.zeros(4, 8, dtype=torch.bfloat16)
    b = torch.zeros(1, 8, 8, dtype=torch.bfloat16)
    c = torch.zeros(4, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _m_grouped_gemm_launch(a, b, c, torch.tensor([4]), True)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        per_token_cast_to_fp8(torch.zeros(2, 128, dtype=torch.bfloat16))
    with pytest.raises(AssertionError):
        _m_grouped_gemm_launch(a, torch.zeros(1, 8, 16, dtype=torch.bfloat16), c, torch.tensor([4]), True)


def test_product_package_does_not_import_the_oracle():
    pkg = ROOT / "triton_grouped_gemm_b200"
    for py in pkg.rglob("*.py"):
        src = py.read_text()
        assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f"{py} imports the oracle"
