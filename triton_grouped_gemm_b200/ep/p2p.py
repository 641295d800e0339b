"""Expert-parallel exchange over peer memory instead of all-to-all collectives.

Every rank owns three buffers of fixed capacity - received fp8 rows, their 1x128 scales, and the
bf16 results of its experts - and maps the other ranks' buffers into its address space (CUDA
IPC through the library's `b200ipc_*` helpers).  Dispatch is then ONE kernel per payload that stores each
(token, k) row straight into the owning rank's receive buffer at its final position (arrival
order: [source rank][local expert] blocks, what the mapped grouped GEMM consumes), and combine is
ONE kernel that loads each (token, k) result from the rank that computed it while it forms the
router-weighted sum.  The bytes cross NVLink once, as plain stores / loads of those kernels; there
is no send-side gather, no staging copy and no permutation.  Ranks synchronise with two one-word
all-reduces per step (rows written -> GEMMs may read; results written -> combine may read).
Positions come from the all-gathered per-expert counts, so every rank computes every offset by
itself.  Plain peer loads / stores only (no multicast objects are involved).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _lib


class _RawCudaBuffer:
    """Device memory owned by the library, visible to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerBuffer:
    """``local``: this rank's [capacity, width] buffer; ``bases``: device pointers of all ranks'
    buffers, each valid in kernels of this rank's GPU (the library's IPC helpers open the other
    ranks' handles with this rank's device current, which also enables peer access)."""

    def __init__(self, capacity_rows: int, width: int, dtype: torch.dtype, device: torch.device, group):
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.capacity = int(capacity_rows)
        self._lib = _lib.load()
        itemsize = torch.empty(0, dtype=dtype).element_size()
        nbytes = self.capacity * width * itemsize
        with torch.cuda.device(device):
            own = ctypes.c_void_p()
            _lib.check(self._lib.b200ipc_alloc(nbytes, ctypes.byref(own)), "b200ipc_alloc")
            self._own_ptr = own.value
            handle = ctypes.create_string_buffer(64)
            _lib.check(self._lib.b200ipc_export(own, handle), "b200ipc_export")
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self._opened = []
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(self._own_ptr)
                    continue
                p = ctypes.c_void_p()
                _lib.check(self._lib.b200ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)), "b200ipc_open")
                self._opened.append(p.value)
                ptrs.append(p.value)
            self._raw = _RawCudaBuffer(self._own_ptr, nbytes)
            self.local = torch.as_tensor(self._raw, device=device).view(dtype).view(self.capacity, width)
        self.bases = (ctypes.c_void_p * self.world)(*ptrs)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def close(self, group=None) -> None:
        """Unmaps the other ranks' buffers, then (after a barrier) frees this rank's."""
        for p in self._opened:
            self._lib.b200ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if dist.is_initialized():
            dist.barrier(group=group)
        if self._own_ptr:
            self.local = None
            self._lib.b200ipc_free(ctypes.c_void_p(self._own_ptr))
            self._own_ptr = 0


@dataclass
class PeerPlan:
    num_tokens: int
    top_k: int
    token_of_pair: torch.Tensor   # [T*k] source token of each pair, in send order (sorted by expert)
    dst_rank: torch.Tensor        # [T*k] int32 owning rank of each pair (send order)
    dst_row: torch.Tensor         # [T*k] int64 row in the owner's buffers (send order)
    pair_rank: torch.Tensor       # [T*k] int32, (token, k) order
    pair_row: torch.Tensor        # [T*k] int64, (token, k) order
    rows_here: int                # rows this rank receives
    block_sizes: torch.Tensor     # [world * e_loc] int64 rows of each [source rank][local expert] block here
    block_expert: torch.Tensor    # [world * e_loc] int32 local expert of each block


def make_peer_plan(topk_idx: torch.Tensor, num_experts: int, group, capacity_rows: int) -> PeerPlan:
    world, me = dist.get_world_size(group), dist.get_rank(group)
    assert num_experts % world == 0
    e_loc = num_experts // world
    t, k = topk_idx.shape
    dev = topk_idx.device
    from .dispatch import route_plan

    flat = topk_idx.reshape(-1).to(torch.int64)
    counts, send_order, pos = route_plan(flat, num_experts)
    counts_flat = torch.empty(world * num_experts, dtype=counts.dtype, device=dev)
    dist.all_gather_into_tensor(counts_flat, counts, group=group)
    counts_all = counts_flat.view(world, num_experts)
    # arrival layout at destination d: blocks (source s, local expert j) in that order
    by_dest = counts_all.view(world, world, e_loc).permute(1, 0, 2).contiguous()      # [d, s, j]
    flat_blocks = by_dest.view(world, world * e_loc)
    starts = (flat_blocks.cumsum(1) - flat_blocks).view(world, world, e_loc)           # [d, s, j]
    dst_block_start = starts[:, me, :].reshape(num_experts)                            # by global expert
    totals = flat_blocks.sum(1).cpu()                                                  # the one host sync
    if int(totals.max()) > capacity_rows:
        raise RuntimeError(f"a rank would receive {int(totals.max())} rows, more than the exchange buffers hold "
                           f"({capacity_rows}); raise capacity_factor")
    my_send_start = counts.cumsum(0) - counts
    e_sorted = flat[send_order]
    dst_rank = (e_sorted // e_loc).to(torch.int32)
    dst_row = dst_block_start[e_sorted] + (torch.arange(t * k, device=dev) - my_send_start[e_sorted])
    return PeerPlan(num_tokens=t, top_k=k, token_of_pair=(send_order // k).contiguous(), dst_rank=dst_rank.contiguous(),
                    dst_row=dst_row.contiguous(), pair_rank=dst_rank[pos].contiguous(), pair_row=dst_row[pos].contiguous(),
                    rows_here=int(totals[me]), block_sizes=by_dest[me].reshape(-1).to(torch.int64).contiguous(),
                    block_expert=torch.arange(e_loc, device=dev, dtype=torch.int32).repeat(world).contiguous())


def scatter_rows(plan: PeerPlan, rows: torch.Tensor, buf: PeerBuffer) -> None:
    """rows [T, width] (one per token) -> every pair's row into its owner's buffer."""
    src = rows.view(torch.uint8) if rows.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else rows
    assert src.is_cuda and src.is_contiguous() and src.dim() == 2
    row_bytes = src.shape[1] * src.element_size()
    assert row_bytes == buf.local.shape[1] * buf.local.element_size()
    with torch.cuda.device(src.device):
        rc = _lib.load().b200moe_scatter_rows_multi(src.data_ptr(), plan.token_of_pair.data_ptr(), buf.bases,
                                                    plan.dst_rank.data_ptr(), plan.dst_row.data_ptr(),
                                                    plan.token_of_pair.numel(), row_bytes, buf.world, buf.capacity,
                                                    _lib.stream_ptr(src.device))
    _lib.check(rc, "b200moe_scatter_rows_multi")


def combine_rows(plan: PeerPlan, buf: PeerBuffer, topk_weight: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_k weight[t,k] * (result row of pair (t,k), read from the rank that computed it)."""
    hidden = buf.local.shape[1]
    out = torch.empty((plan.num_tokens, hidden), dtype=torch.bfloat16, device=buf.local.device)
    w32 = topk_weight.reshape(-1).to(torch.float32).contiguous()
    with torch.cuda.device(out.device):
        rc = _lib.load().b200moe_combine_topk_multi(buf.bases, plan.pair_rank.data_ptr(), plan.pair_row.data_ptr(),
                                                    w32.data_ptr(), out.data_ptr(), plan.num_tokens, plan.top_k, hidden,
                                                    buf.world, buf.capacity, _lib.stream_ptr(out.device))
    _lib.check(rc, "b200moe_combine_topk_multi")
    return out


@dataclass
class PeerChunkPlan:
    """Peer-memory plan split into ``chunks`` groups of local experts (chunk c = local experts
    [c*ec, (c+1)*ec) on every rank).  Send order and every rank's receive buffers are chunk-major:
    [chunk][source rank][expert of the chunk], so a chunk is one contiguous row range everywhere."""
    num_tokens: int
    top_k: int
    chunks: int
    token_of_pair: torch.Tensor      # [T*k] send order
    dst_rank: torch.Tensor           # [T*k] int32
    dst_row: torch.Tensor            # [T*k] int64
    pos: torch.Tensor                # [T*k] position of pair (t, k) in send order = its row in this rank's return buffer
    send_offsets: List[int]          # [chunks + 1] send-order ranges of the chunks
    recv_offsets: List[int]          # [chunks + 1] row ranges of the chunks in this rank's receive buffers
    block_sizes: List[torch.Tensor]  # per chunk [world * ec] int64
    block_expert: List[torch.Tensor] # per chunk [world * ec] int32 (local expert index)
    meta: torch.Tensor               # [T*k, 2] int64: (send-order position, this rank) of each pair


def make_peer_chunk_plan(topk_idx: torch.Tensor, num_experts: int, group, capacity_rows: int,
                         chunks: int) -> PeerChunkPlan:
    from .dispatch import route_plan

    world, me = dist.get_world_size(group), dist.get_rank(group)
    assert num_experts % world == 0
    e_loc = num_experts // world
    assert e_loc % chunks == 0
    ec = e_loc // chunks
    t, k = topk_idx.shape
    n = t * k
    dev = topk_idx.device
    flat = topk_idx.reshape(-1).to(torch.int64)
    rank_of = flat // e_loc
    local = flat - rank_of * e_loc
    chunk_of = local // ec
    key = chunk_of * (world * ec) + rank_of * ec + (local - chunk_of * ec)
    counts_by_key, send_order, pos = route_plan(key, num_experts)
    e_ids = torch.arange(num_experts, device=dev)
    key_of_expert = ((e_ids % e_loc) // ec) * (world * ec) + (e_ids // e_loc) * ec + (e_ids % e_loc) % ec
    counts = counts_by_key[key_of_expert]                                             # by global expert
    counts_flat = torch.empty(world * num_experts, dtype=counts.dtype, device=dev)
    dist.all_gather_into_tensor(counts_flat, counts, group=group)
    # arrival layout at destination d: blocks (chunk c, source s, expert j of the chunk) in that order
    by_dest = counts_flat.view(world, world, chunks, ec).permute(1, 2, 0, 3).contiguous()   # [d, c, s, j]
    flat_blocks = by_dest.view(world, chunks * world * ec)
    starts = (flat_blocks.cumsum(1) - flat_blocks).view(world, chunks, world, ec)            # [d, c, s, j]
    dst_block_start = starts[:, :, me, :].reshape(num_experts)                               # (d, c, j) = global expert
    totals = flat_blocks.sum(1)
    host = torch.cat([totals, by_dest[me].sum((1, 2)), counts_by_key.view(chunks, world * ec).sum(1)]).cpu()  # one sync
    if int(host[:world].max()) > capacity_rows:
        raise RuntimeError(f"a rank would receive {int(host[:world].max())} rows, more than the exchange buffers hold "
                           f"({capacity_rows}); raise capacity_factor")
    recv_offsets, send_offsets = [0], [0]
    for c in range(chunks):
        recv_offsets.append(recv_offsets[-1] + int(host[world + c]))
        send_offsets.append(send_offsets[-1] + int(host[world + chunks + c]))
    send_start_by_key = counts_by_key.cumsum(0) - counts_by_key
    key_sorted = key[send_order]
    e_sorted = flat[send_order]
    idx = torch.arange(n, device=dev)
    dst_rank = (e_sorted // e_loc).to(torch.int32)
    dst_row = dst_block_start[e_sorted] + (idx - send_start_by_key[key_sorted])
    meta = torch.stack([idx, torch.full_like(idx, me)], dim=1).contiguous()
    return PeerChunkPlan(num_tokens=t, top_k=k, chunks=chunks, token_of_pair=(send_order // k).contiguous(),
                         dst_rank=dst_rank.contiguous(), dst_row=dst_row.contiguous(), pos=pos,
                         send_offsets=send_offsets, recv_offsets=recv_offsets,
                         block_sizes=[by_dest[me, c].reshape(-1).to(torch.int64).contiguous() for c in range(chunks)],
                         block_expert=[(torch.arange(ec, device=dev, dtype=torch.int32) + c * ec).repeat(world).contiguous()
                                       for c in range(chunks)],
                         meta=meta)


def scatter_range(src: torch.Tensor, src_idx: torch.Tensor, dst_rank: torch.Tensor, dst_row: torch.Tensor,
                  buf: PeerBuffer) -> None:
    """buf[dst_rank[i]][dst_row[i]] = src[src_idx[i]] for the given index vectors (contiguous tensors
    that the caller keeps alive until the stream has run the kernel)."""
    src2 = src.view(torch.uint8) if src.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else src
    assert src2.is_contiguous() and src_idx.is_contiguous() and dst_rank.is_contiguous() and dst_row.is_contiguous()
    row_bytes = src2.shape[1] * src2.element_size()
    assert row_bytes == buf.local.shape[1] * buf.local.element_size()
    with torch.cuda.device(src2.device):
        rc = _lib.load().b200moe_scatter_rows_multi(src2.data_ptr(), src_idx.data_ptr(), buf.bases, dst_rank.data_ptr(),
                                                    dst_row.data_ptr(), src_idx.numel(), row_bytes, buf.world,
                                                    buf.capacity, _lib.stream_ptr(src2.device))
    _lib.check(rc, "b200moe_scatter_rows_multi")
