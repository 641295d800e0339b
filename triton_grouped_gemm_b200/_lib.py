"""ctypes binding of libb200gemm.so (the C ABI declared in include/b200gemm.h).

There is no fallback: if the library cannot be loaded, or a call fails, a RuntimeError is
raised -- nothing in this package computes on the CPU or through another GEMM library.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_int, c_int64, c_void_p, c_uint, POINTER, c_float
from pathlib import Path

import torch

import os

PKG = Path(__file__).resolve().parent
# B200GEMM_LIBRARY overrides the in-tree library (e.g. a build with different tuning).
LIB_PATH = Path(os.environ["B200GEMM_LIBRARY"]) if os.environ.get("B200GEMM_LIBRARY") else PKG / "libb200gemm.so"

_lock = threading.Lock()
_lib = None

# name -> argtypes; every function returns int except where noted
_SIGNATURES = {
    "b200gemm_version": [],
    "b200gemm_device_status": [POINTER(c_uint), c_int],
    "b200gemm_sm_count": [],
    "b200gemm_set_block_n": [c_int],
    "b200gemm_set_cta_pair": [c_int],
    "b200gemm_cta_pair_grid": [],
    "b200gemm_m_grouped": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int, c_int,
                           c_int, c_void_p],
    "b200gemm_m_grouped_padded": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int,
                                  c_int, c_int, c_void_p],
    "b200gemm_m_grouped_masked": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_int, c_void_p],
    "b200gemm_k_grouped": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
                           c_int, c_void_p, c_int64, c_int, c_void_p],
    "b200gemm_k_grouped_static_scratch": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                          c_int64, c_int, c_int, c_int, c_int, c_void_p],
    "b200gemm_fp8_m_grouped_rowcol": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "b200gemm_fp8_k_grouped_rowcol": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64,
                                      c_int, c_int, c_int, c_int, c_void_p, c_int64, c_int, c_void_p],
    "b200gemm_fp8_m_grouped_block": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64,
                                     c_int, c_int, c_int, c_int, c_void_p],
    "b200gemm_fp8_m_grouped_block_mapped": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p],
    "b200gemm_fp8_m_grouped_block_swiglu": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                            c_int, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p],
    "b200gemm_fp8_m_grouped_masked_block": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_int, c_int, c_int, c_int, c_void_p],
    "b200gemm_fp8_k_grouped_block": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64,
                                     c_int, c_int, c_void_p, c_int64, c_int, c_void_p],
    "b200moe_route_plan": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200moe_route_plan_mapped": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200moe_peer_plan": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int64, c_int, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200moe_scatter_rows_multi": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64,
                                   c_int64, c_int, c_void_p],
    "b200moe_dispatch_quant_rows_multi": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                          c_int64, c_int64, c_int, c_int, c_int, c_int64, c_int, c_int, c_void_p],
    "b200moe_dispatch_rows_multi": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                    c_int64, c_int64, c_int, c_int, c_int64, c_int, c_int, c_void_p],
    "b200moe_return_rows_multi": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_int, c_void_p],
    "b200moe_combine_topk_multi": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                   c_int64, c_void_p],
    "b200ipc_alloc": [c_int64, c_void_p],
    "b200ipc_free": [c_void_p],
    "b200ipc_export": [c_void_p, c_void_p],
    "b200ipc_open": [c_void_p, c_void_p],
    "b200ipc_close": [c_void_p],
    "b200ipc_copy_many_async": [c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200layout_group_starts": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "b200layout_psum": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "b200layout_grouped_rows": [c_void_p, c_int, c_int, c_int, c_void_p, c_int64, c_void_p],
    "b200moe_gather_rows": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p],
    "b200moe_quant_scatter_rows": [c_void_p, c_int, c_int64, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p],
    "b200moe_combine_topk": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_void_p],
    "b200quant_act_1x128": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p],
    "b200quant_swiglu_act_1x128": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p],
    "b200quant_w_128x128": [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p],
    "b200quant_trans_expand_128x": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                    c_int64, c_int, c_void_p],
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES) + ("b200gemm_last_error", "b200gemm_k_grouped_workspace_bytes")


def load():
    """Load (once) and return the ctypes library; build it in-tree if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            from . import build as _build

            _build.build()
        try:
            lib = ctypes.CDLL(str(LIB_PATH))
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise RuntimeError(f"cannot load {LIB_PATH}: {exc}") from exc
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        lib.b200gemm_last_error.argtypes = []
        lib.b200gemm_last_error.restype = c_char_p
        lib.b200gemm_k_grouped_workspace_bytes.argtypes = [c_int]
        lib.b200gemm_k_grouped_workspace_bytes.restype = ctypes.c_longlong
        _lib = lib
    return _lib


def last_error() -> str:
    return load().b200gemm_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with status {rc}: {last_error()}")


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(
                "the b200 backend runs only on CUDA tensors (sm_100a); there is no CPU fallback "
                f"(got a tensor on {t.device})"
            )


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor) -> int:
    return t.data_ptr()


def device_status(clear: bool = True) -> int:
    """Synchronise the current device and return its status word (0 = no device-side error)."""
    out = c_uint(0)
    check(load().b200gemm_device_status(ctypes.byref(out), 1 if clear else 0), "b200gemm_device_status")
    return int(out.value)


def k_grouped_workspace(num_groups: int, device: torch.device):
    """Scratch for the balanced K-grouped scheduler, from torch's stream-ordered allocator (a
    fresh buffer per call, so calls on different streams never share one).  None when the group
    count exceeds what the scheduler supports (the kernel then assigns tiles round-robin)."""
    if num_groups > 4096:
        return None, 0
    nbytes = int(load().b200gemm_k_grouped_workspace_bytes(num_groups))
    return torch.empty(nbytes, dtype=torch.uint8, device=device), nbytes


def dtype_code(dtype: torch.dtype) -> int:
    code = {torch.bfloat16: 0, torch.float16: 1}.get(dtype, -1)
    assert code >= 0, f"data type {dtype} not supported"
    return code


def sizes_arg(sizes: torch.Tensor):
    """Group sizes stay on the device; int32 and int64 are passed through untouched."""
    assert sizes.dim() == 1, "size_per_group must be 1D"
    if sizes.dtype not in (torch.int32, torch.int64):
        sizes = sizes.to(torch.int64)
    if not sizes.is_contiguous():
        sizes = sizes.contiguous()
    return sizes, 1 if sizes.dtype == torch.int64 else 0
