"""Backend selection (mirror of the reference's gemm/backends.py:12-68).

The reference's ``'triton'`` backend is replaced by ``'b200'``: hand-written sm_100a CUDA
behind a C ABI.  ``'deep_gemm'`` stays selectable for callers that have that package;
``'auto'`` resolves to ``'b200'``.
"""

from __future__ import annotations

import importlib.util
from enum import Enum
from typing import Optional, Tuple

import torch


class GemmBackend(str, Enum):
    AUTO = "auto"
    B200 = "b200"
    DEEP_GEMM = "deep_gemm"


_ALIASES = {"deepgemm": "deep_gemm", "deep-gemm": "deep_gemm", "sm100": "b200", "sm_100a": "b200"}


def normalize_backend(backend) -> GemmBackend:
    if isinstance(backend, GemmBackend):
        return backend
    name = _ALIASES.get(backend, backend)
    try:
        return GemmBackend(name)
    except ValueError as exc:
        valid = ", ".join(item.value for item in GemmBackend)
        raise ValueError(f"Unsupported GEMM backend {name!r}; expected one of: {valid}") from exc


def is_deep_gemm_available() -> bool:
    return importlib.util.find_spec("deep_gemm") is not None


def current_cuda_arch() -> Optional[Tuple[int, int]]:
    try:
        if not torch.cuda.is_available():
            return None
        return torch.cuda.get_device_capability()
    except Exception:
        return None


def deep_gemm_supports_current_device() -> bool:
    arch = current_cuda_arch()
    return arch is not None and arch[0] in (9, 10)


def is_b200_available() -> bool:
    """True when the CUDA extension loads and the current device is compute capability 10.x."""
    arch = current_cuda_arch()
    if arch is None or arch[0] != 10:
        return False
    try:
        from .. import _lib

        _lib.load()
        return True
    except Exception:
        return False


def select_backend(backend=GemmBackend.AUTO) -> GemmBackend:
    backend = normalize_backend(backend)
    if backend != GemmBackend.AUTO:
        return backend
    return GemmBackend.B200


def require_b200_support() -> None:
    arch = current_cuda_arch()
    if arch is None or arch[0] != 10:
        text = "no CUDA device" if arch is None else f"SM{arch[0]}{arch[1]}"
        raise RuntimeError(f"b200 backend requested, but current device is unsupported ({text})")
    from .. import _lib

    _lib.load()


def require_deep_gemm_support() -> None:
    if not is_deep_gemm_available():
        raise RuntimeError("DeepGEMM backend requested, but Python package 'deep_gemm' is not installed")
    if not deep_gemm_supports_current_device():
        arch = current_cuda_arch()
        arch_text = "no CUDA device" if arch is None else f"SM{arch[0]}{arch[1]}"
        raise RuntimeError(f"DeepGEMM backend requested, but current device is unsupported ({arch_text})")
