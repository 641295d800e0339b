"""Grouped GEMM for callers whose operands live in host memory.

``m_grouped_gemm_host`` takes (ideally pinned) host tensors and returns a host tensor.  The
groups are cut into a few chunks and three CUDA streams pipeline them: while chunk i is being
multiplied, chunk i+1 is on its way to the device and the result of chunk i-1 on its way back,
so the call costs about as much as the slower PCIe direction alone instead of
H2D + GEMM + D2H one after the other.  The arithmetic is the M-grouped kernel, one launch per
chunk; results are bit-identical to a single launch (rows are independent).
"""

from __future__ import annotations

from typing import Optional

import torch

from .gemm.BF16.m_grouped_gemm_TMA import _m_grouped_gemm_launch


def _chunk_bounds(sizes_host: torch.Tensor, chunks: int):
    """Split [0, G) into at most `chunks` ranges of roughly equal row count."""
    total = int(sizes_host.sum())
    g = sizes_host.numel()
    target = max(total // max(chunks, 1), 1)
    bounds, acc, start = [], 0, 0
    for i, s in enumerate(sizes_host.tolist()):
        acc += s
        if acc >= target and i + 1 < g and len(bounds) + 1 < chunks:
            bounds.append((start, i + 1))
            start, acc = i + 1, 0
    bounds.append((start, g))
    return bounds


def m_grouped_gemm_host(a_host: torch.Tensor, b_host: torch.Tensor, size_per_group: torch.Tensor,
                        trans_b: bool = False, out_host: Optional[torch.Tensor] = None, chunks: int = 8,
                        device: Optional[torch.device] = None) -> torch.Tensor:
    """a_host [M, K], b_host [G, N, K] (trans_b) or [G, K, N], size_per_group [G] on the host.
    Returns C [M, N] on the host (pinned if ``out_host`` is None)."""
    assert not a_host.is_cuda and not b_host.is_cuda and not size_per_group.is_cuda, "operands must be host tensors"
    if not torch.cuda.is_available():
        raise RuntimeError("the b200 backend needs a CUDA device; there is no CPU fallback")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    sizes_host = size_per_group.to(torch.int64)
    m, k = a_host.shape
    n = b_host.shape[1] if trans_b else b_host.shape[2]
    if out_host is None:
        out_host = torch.empty((m, n), dtype=a_host.dtype).pin_memory()
    starts = torch.cumsum(sizes_host, 0) - sizes_host
    a_dev = torch.empty((m, k), dtype=a_host.dtype, device=dev)
    b_dev = torch.empty(b_host.shape, dtype=b_host.dtype, device=dev)
    c_dev = torch.empty((m, n), dtype=a_host.dtype, device=dev)
    sizes_dev = sizes_host.to(dev, non_blocking=True)
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    for g0, g1 in _chunk_bounds(sizes_host, chunks):
        r0 = int(starts[g0])
        r1 = int(starts[g1 - 1] + sizes_host[g1 - 1])
        with torch.cuda.stream(s_in):
            a_dev[r0:r1].copy_(a_host[r0:r1], non_blocking=True)
            b_dev[g0:g1].copy_(b_host[g0:g1], non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(s_in)
        main.wait_event(ready)
        if r1 > r0:
            _m_grouped_gemm_launch(a_dev[r0:r1], b_dev[g0:g1], c_dev[r0:r1], sizes_dev[g0:g1], trans_b)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            out_host[r0:r1].copy_(c_dev[r0:r1], non_blocking=True)
    main.wait_stream(s_out)
    # keep the device buffers alive until the side streams are done with them
    for t in (a_dev, b_dev, c_dev):
        t.record_stream(s_in)
        t.record_stream(s_out)
    return out_host
