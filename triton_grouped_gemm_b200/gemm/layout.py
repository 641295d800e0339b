"""Integer layouts of grouped GEMM problems (mirror of the reference's gemm/layout.py:11-126).

Same names, arguments, results and ValueErrors as the reference.  Two differences in how the
results are produced: for sizes on a CUDA device the group starts, the per-row and the psum
layouts come from the library's layout kernels (the reference loops over ``.tolist()`` on the
host; host tensors are handled with tensor ops, as integer host helpers), and
``device_group_metadata`` gives the kernels' view of a size vector for debugging -- the CUDA
kernels themselves derive all of this on the fly from ``size_per_group``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence, Union

import torch

SizesLike = Union[torch.Tensor, Sequence[int]]


@dataclass(frozen=True)
class GroupedLayout:
    starts: torch.Tensor
    sizes: torch.Tensor
    padded_sizes: torch.Tensor

    @property
    def total_m(self) -> torch.Tensor:
        return self.sizes.sum()

    @property
    def total_padded_m(self) -> torch.Tensor:
        return self.padded_sizes.sum()


def as_group_sizes(size_per_group: SizesLike, *, device=None, dtype: torch.dtype = torch.int32) -> torch.Tensor:
    """Validated, contiguous 1-D size vector (ValueError on wrong rank, empty, negative)."""
    if isinstance(size_per_group, torch.Tensor):
        sizes = size_per_group if device is None else size_per_group.to(device=device)
        sizes = sizes.to(dtype=dtype)
    else:
        sizes = torch.tensor(size_per_group, device=device, dtype=dtype)
    if sizes.dim() != 1:
        raise ValueError(f"size_per_group must be 1D, got shape {tuple(sizes.shape)}")
    if sizes.numel() == 0:
        raise ValueError("size_per_group must contain at least one group")
    if bool((sizes < 0).any().item()):
        raise ValueError("size_per_group cannot contain negative sizes")
    return sizes.contiguous()


def round_up_to_alignment(sizes: torch.Tensor, alignment: int) -> torch.Tensor:
    if alignment <= 0:
        raise ValueError(f"alignment must be positive, got {alignment}")
    return torch.div(sizes + (alignment - 1), alignment, rounding_mode="floor") * alignment


def _exclusive_cumsum(v: torch.Tensor) -> torch.Tensor:
    return v.cumsum(0) - v


def make_grouped_layout(size_per_group: SizesLike, block_m: int = 128) -> GroupedLayout:
    sizes = as_group_sizes(size_per_group)
    padded = round_up_to_alignment(sizes, block_m)
    return GroupedLayout(starts=_exclusive_cumsum(padded).contiguous(), sizes=sizes, padded_sizes=padded.contiguous())


def _on_device(sizes: torch.Tensor) -> bool:
    return sizes.is_cuda


def _sizes_ptr(sizes: torch.Tensor):
    """(contiguous int32/int64 tensor, is_int64) for the C ABI."""
    if sizes.dtype not in (torch.int32, torch.int64):
        sizes = sizes.to(torch.int64)
    return sizes.contiguous(), int(sizes.dtype == torch.int64)


def make_group_starts(size_per_group: SizesLike, *, padded: bool = False, block_m: int = 128,
                      dtype: torch.dtype = torch.int32) -> torch.Tensor:
    sizes = as_group_sizes(size_per_group, dtype=dtype)
    if _on_device(sizes) and dtype == torch.int32:
        from .. import _lib

        if block_m <= 0:
            raise ValueError(f"alignment must be positive, got {block_m}")
        s, is64 = _sizes_ptr(sizes)
        out = torch.empty(s.numel(), dtype=torch.int32, device=s.device)
        with torch.cuda.device(s.device):
            rc = _lib.load().b200layout_group_starts(s.data_ptr(), is64, s.numel(), int(padded), int(block_m),
                                                     out.data_ptr(), _lib.stream_ptr(s.device))
        _lib.check(rc, "b200layout_group_starts")
        return out
    if padded:
        sizes = round_up_to_alignment(sizes, block_m)
    return _exclusive_cumsum(sizes).contiguous()


def make_deep_gemm_grouped_layout(size_per_group: SizesLike, *, block_m: int = 128, device=None) -> torch.Tensor:
    """One int32 per padded M row: the expert id on real rows, -1 on padding rows.  The length of
    the result is data dependent, so this call synchronises the host once (``.item()``) to size
    it, as the reference does (gemm/layout.py:73-98); the rows themselves are written by a kernel
    when the sizes live on the device."""
    sizes = as_group_sizes(size_per_group, device=device, dtype=torch.int32)
    padded = round_up_to_alignment(sizes, block_m).to(torch.int64)
    total = int(padded.sum().item())
    if _on_device(sizes):
        from .. import _lib

        s, is64 = _sizes_ptr(sizes)
        out = torch.empty(total, dtype=torch.int32, device=s.device)
        with torch.cuda.device(s.device):
            rc = _lib.load().b200layout_grouped_rows(s.data_ptr(), is64, s.numel(), int(block_m), out.data_ptr(), total,
                                                     _lib.stream_ptr(s.device))
        _lib.check(rc, "b200layout_grouped_rows")
        return out
    ids = torch.arange(sizes.numel(), device=sizes.device, dtype=torch.int32)
    row_group = torch.repeat_interleave(ids, padded, output_size=total)
    starts = _exclusive_cumsum(padded)
    local = torch.arange(total, device=sizes.device, dtype=torch.int64) - starts[row_group.long()]
    pad_row = local >= sizes.to(torch.int64)[row_group.long()]
    return torch.where(pad_row, torch.full_like(row_group, -1), row_group).contiguous()


def make_deep_gemm_psum_layout(size_per_group: SizesLike, *, block_m: int = 128, device=None) -> torch.Tensor:
    """Per expert: the end offset of its real rows in padded-M coordinates."""
    sizes = as_group_sizes(size_per_group, device=device, dtype=torch.int32)
    if _on_device(sizes):
        from .. import _lib

        if block_m <= 0:
            raise ValueError(f"alignment must be positive, got {block_m}")
        s, is64 = _sizes_ptr(sizes)
        out = torch.empty(s.numel(), dtype=torch.int32, device=s.device)
        with torch.cuda.device(s.device):
            rc = _lib.load().b200layout_psum(s.data_ptr(), is64, s.numel(), int(block_m), out.data_ptr(),
                                             _lib.stream_ptr(s.device))
        _lib.check(rc, "b200layout_psum")
        return out
    padded = round_up_to_alignment(sizes, block_m)
    return (_exclusive_cumsum(padded) + sizes).to(torch.int32).contiguous()


def validate_total_m(size_per_group: SizesLike, total_m: int) -> None:
    actual = int(as_group_sizes(size_per_group, dtype=torch.int64).sum().item())
    if actual != total_m:
        raise ValueError(f"sum(size_per_group) must equal M ({total_m}), got {actual}")


def device_group_metadata(size_per_group: torch.Tensor, block_m: int = 128):
    """(pad_start, pad_end, group_start, group_end, m_indices_pad, M_pad) -- the tuple the
    reference's ``_build_m_grouped_metadata`` returns (gemm/BF16/m_grouped_gemm_TMA.py:297-326).
    Kept for benchmark code that builds it and passes it as ``metadata=``; the B200 kernels never
    read it.  Like the reference it synchronises the host once (``.item()``, to size
    ``m_indices_pad``) - the GEMM entry points themselves do not call it and do not synchronise."""
    s = size_per_group.to(torch.int32)
    p = round_up_to_alignment(s, block_m)
    pad_end = p.cumsum(0).to(torch.int32)
    pad_start = pad_end - p
    group_end = s.cumsum(0).to(torch.int32)
    group_start = group_end - s
    m_total = int(size_per_group.sum().item())
    g = s.numel()
    cap = m_total // block_m + g
    tiles = (p // block_m).to(torch.int64)
    idx = torch.repeat_interleave(torch.arange(g, device=s.device, dtype=torch.int32), tiles)
    m_indices_pad = torch.zeros(cap, device=s.device, dtype=torch.int32)
    m_indices_pad[: idx.numel()] = idx
    return pad_start, pad_end, group_start, group_end, m_indices_pad, p.sum()
