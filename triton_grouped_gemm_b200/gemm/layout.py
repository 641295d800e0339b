"""Integer layouts of grouped GEMM problems (mirror of the reference's gemm/layout.py:11-126).

Same names, arguments, results and ValueErrors as the reference.  Two differences in how the
results are produced: the per-row and psum layouts are built with tensor ops on the device
that holds the sizes (the reference loops over ``.tolist()`` on the host), and
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


def make_group_starts(size_per_group: SizesLike, *, padded: bool = False, block_m: int = 128,
                      dtype: torch.dtype = torch.int32) -> torch.Tensor:
    sizes = as_group_sizes(size_per_group, dtype=dtype)
    if padded:
        sizes = round_up_to_alignment(sizes, block_m)
    return _exclusive_cumsum(sizes).contiguous()


def make_deep_gemm_grouped_layout(size_per_group: SizesLike, *, block_m: int = 128, device=None) -> torch.Tensor:
    """One int32 per padded M row: the expert id on real rows, -1 on padding rows."""
    sizes = as_group_sizes(size_per_group, device=device, dtype=torch.int32)
    padded = round_up_to_alignment(sizes, block_m).to(torch.int64)
    total = int(padded.sum().item())
    ids = torch.arange(sizes.numel(), device=sizes.device, dtype=torch.int32)
    row_group = torch.repeat_interleave(ids, padded, output_size=total)
    starts = _exclusive_cumsum(padded)
    local = torch.arange(total, device=sizes.device, dtype=torch.int64) - starts[row_group.long()]
    pad_row = local >= sizes.to(torch.int64)[row_group.long()]
    return torch.where(pad_row, torch.full_like(row_group, -1), row_group).contiguous()


def make_deep_gemm_psum_layout(size_per_group: SizesLike, *, block_m: int = 128, device=None) -> torch.Tensor:
    """Per expert: the end offset of its real rows in padded-M coordinates."""
    sizes = as_group_sizes(size_per_group, device=device, dtype=torch.int32)
    padded = round_up_to_alignment(sizes, block_m)
    return (_exclusive_cumsum(padded) + sizes).to(torch.int32).contiguous()


def validate_total_m(size_per_group: SizesLike, total_m: int) -> None:
    actual = int(as_group_sizes(size_per_group, dtype=torch.int64).sum().item())
    if actual != total_m:
        raise ValueError(f"sum(size_per_group) must equal M ({total_m}), got {actual}")


def device_group_metadata(size_per_group: torch.Tensor, block_m: int = 128):
    """(pad_start, pad_end, group_start, group_end, m_indices_pad, M_pad) -- the tuple the
    reference's ``_build_m_grouped_metadata`` returns (gemm/BF16/m_grouped_gemm_TMA.py:297-326),
    built without a host synchronisation except for sizing ``m_indices_pad``."""
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
