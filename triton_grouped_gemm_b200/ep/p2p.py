"""Expert-parallel exchange over peer memory instead of all-to-all collectives.

Every rank owns three buffers of fixed capacity - received fp8 rows, their 1x128 scales, and the
bf16 results of its experts - and maps the other ranks' buffers into its address space (CUDA
IPC through the library's `b200ipc_*` helpers).  Dispatch is then ONE kernel per payload that stores each
(token, k) row straight into the owning rank's receive buffer at its final position
([local expert][source rank] order: every expert's rows are contiguous, so the grouped GEMM sees
one row group per expert whatever the number of ranks), and combine is
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
        """Unmaps the other ranks' buffers, then (after a barrier) frees this rank's.  Collective:
        every rank of the group must call it, with no kernel that touches the buffers in flight."""
        if not self._own_ptr and not self._opened:
            return
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
    size_per_group: torch.Tensor  # [e_loc] int64 rows of each local expert here (all source ranks together)


def _arrival_layout(counts: torch.Tensor, group, num_experts: int):
    """All-gathers the per-expert pair counts and lays every rank's receive buffer out as
    [local expert][source rank] blocks.  Returns (by_dest [d, l, s] block sizes, dst_block_start
    [num_experts]: where THIS rank's rows for each global expert start in the owner's buffer,
    totals [world]: rows every rank receives)."""
    world, me = dist.get_world_size(group), dist.get_rank(group)
    e_loc = num_experts // world
    counts_flat = torch.empty(world * num_experts, dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(counts_flat, counts.contiguous(), group=group)
    by_dest = counts_flat.view(world, world, e_loc).permute(1, 2, 0).contiguous()       # [d, l, s]
    flat_blocks = by_dest.view(world, e_loc * world)
    starts = (flat_blocks.cumsum(1) - flat_blocks).view(world, e_loc, world)            # [d, l, s]
    return by_dest, starts[:, :, me].reshape(num_experts), flat_blocks.sum(1)


def make_peer_plan(topk_idx: torch.Tensor, num_experts: int, group, capacity_rows: int) -> PeerPlan:
    world, me = dist.get_world_size(group), dist.get_rank(group)
    assert num_experts % world == 0
    e_loc = num_experts // world
    t, k = topk_idx.shape
    dev = topk_idx.device
    from .dispatch import route_plan

    flat = topk_idx.reshape(-1).to(torch.int64)
    counts, send_order, pos = route_plan(flat, num_experts)
    by_dest, dst_block_start, totals_dev = _arrival_layout(counts, group, num_experts)
    totals = torch.cat([totals_dev, counts.sum()[None]]).cpu()                         # the one host sync
    if int(totals[:world].max()) > capacity_rows:
        raise RuntimeError(f"a rank would receive {int(totals[:world].max())} rows, more than the exchange buffers "
                           f"hold ({capacity_rows}); raise capacity_factor")
    my_send_start = counts.cumsum(0) - counts
    valid = send_order[:int(totals[world])]            # pairs with an expert id out of range are not sent
    e_sorted = flat[valid]
    dst_rank = (e_sorted // e_loc).to(torch.int32)
    dst_row = dst_block_start[e_sorted] + (torch.arange(valid.numel(), device=dev) - my_send_start[e_sorted])
    ok = pos >= 0
    safe = pos.clamp(min=0)
    pair_rank = torch.where(ok, dst_rank[safe], torch.full_like(dst_rank[safe], -1))   # -1: skipped by the combine
    pair_row = torch.where(ok, dst_row[safe], torch.full_like(dst_row[safe], -1))
    return PeerPlan(num_tokens=t, top_k=k, token_of_pair=(valid // k).contiguous(), dst_rank=dst_rank.contiguous(),
                    dst_row=dst_row.contiguous(), pair_rank=pair_rank.contiguous(), pair_row=pair_row.contiguous(),
                    rows_here=int(totals[me]), size_per_group=by_dest[me].sum(-1).to(torch.int64).contiguous())


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
                                                    src.shape[0], 0, _lib.stream_ptr(src.device))
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
    """Peer-memory plan split into chunks of consecutive local experts (chunk c = local experts
    [bounds[c], bounds[c+1]) on every rank).  Send order is chunk-major ([chunk][destination
    rank][expert]); every rank's receive buffers are [local expert][source rank], so a chunk is one
    contiguous row range everywhere and each of its experts is one contiguous row group."""
    num_tokens: int
    top_k: int
    bounds: List[int]                # [chunks + 1] local-expert boundaries of the chunks
    token_of_pair: torch.Tensor      # [T*k] send order
    dst_rank: torch.Tensor           # [T*k] int32
    dst_row: torch.Tensor            # [T*k] int64
    pos: torch.Tensor                # [T*k] position of pair (t, k) in send order = its row in this rank's return buffer
    send_offsets: List[int]          # [chunks + 1] send-order ranges of the chunks
    recv_offsets: List[int]          # [chunks + 1] row ranges of the chunks in this rank's receive buffers
    size_per_group: torch.Tensor     # [e_loc] int64 rows of each local expert here
    blk_count: "object" = None       # host int array [e_loc, world]: rows of block (local expert, source rank) here
    blk_start: "object" = None       # host int array [e_loc, world]: first row of that block in this rank's buffers
    ret_row0: "object" = None        # host int array [e_loc, world]: first row of that block in the SOURCE's return buffer
    snd_count: "object" = None       # host int array [world, e_loc]: pairs this rank sends to expert l of rank d
    snd_src0: "object" = None        # host int array [world, e_loc]: where they start in this rank's send order
    snd_dst0: "object" = None        # host int array [world, e_loc]: first row of that block in rank d's buffers

    @property
    def chunks(self) -> int:
        return len(self.bounds) - 1


def chunk_bounds(e_loc: int, chunks: int, taper: bool = False) -> List[int]:
    """Boundaries of `chunks` runs of consecutive local experts: nearly equal, or - ``taper`` -
    with a first and a last run of about half the size of the others (the first dispatch and the
    last return of a pipelined step have nothing to hide behind, so they are kept short)."""
    chunks = max(1, min(chunks, e_loc))
    if not taper or chunks < 3 or e_loc < 2 * chunks:
        return [(c * e_loc) // chunks for c in range(chunks + 1)]
    # weights 1, 2, 2, ..., 2, 1 over the runs
    total = 2 * (chunks - 1)
    acc, bounds = 0, [0]
    for c in range(chunks):
        acc += 1 if c in (0, chunks - 1) else 2
        b = max(bounds[-1] + 1, min(e_loc - (chunks - 1 - c), round(acc * e_loc / total)))
        bounds.append(b)
    bounds[-1] = e_loc
    return bounds


_KEY_TABLES = {}


def _key_tables(world: int, e_loc: int, bounds: tuple, dev):
    """Sort key of global expert (rank r, local expert l) = its place in (chunk of l, r, l) order, so
    that the send order is chunk-major and, inside a chunk, grouped by destination rank, then
    expert.  Returns (key_of_expert on the host, its inverse on the host, key_of_expert on ``dev``,
    the inverse on ``dev`` as int32); cached, the tables depend only on the layer's shape."""
    ck = (world, e_loc, bounds, str(dev))
    if ck not in _KEY_TABLES:
        import numpy as np

        b = np.asarray(bounds)
        l_ids = np.arange(e_loc)
        chunk_of_l = np.searchsorted(b[1:], l_ids, side="right")
        width = (b[1:] - b[:-1])[chunk_of_l]
        key_rl = (world * b[:-1][chunk_of_l])[None, :] + np.arange(world)[:, None] * width[None, :] \
            + (l_ids - b[:-1][chunk_of_l])[None, :]                        # [r, l]
        key_h = key_rl.reshape(world * e_loc).astype(np.int64)
        inv_h = np.argsort(key_h)
        _KEY_TABLES[ck] = (key_h, inv_h, torch.from_numpy(key_h).to(dev), torch.from_numpy(inv_h.astype(np.int32)).to(dev))
    return _KEY_TABLES[ck]


def make_peer_chunk_plan(topk_idx: torch.Tensor, num_experts: int, group, capacity_rows: int,
                         bounds: List[int]) -> PeerChunkPlan:
    from .dispatch import route_plan

    world, me = dist.get_world_size(group), dist.get_rank(group)
    assert num_experts % world == 0
    e_loc = num_experts // world
    chunks = len(bounds) - 1
    assert bounds[0] == 0 and bounds[-1] == e_loc and all(bounds[c] < bounds[c + 1] for c in range(chunks))
    t, k = topk_idx.shape
    n = t * k
    dev = topk_idx.device
    flat = topk_idx.reshape(-1).to(torch.int64)
    key_of_expert_h, expert_of_key, key_of_expert, expert_of_key_dev = _key_tables(world, e_loc, tuple(bounds), dev)
    if flat.is_cuda:
        return _make_peer_chunk_plan_cuda(flat, t, k, num_experts, group, capacity_rows, list(bounds), key_of_expert_h,
                                          expert_of_key, key_of_expert, expert_of_key_dev)
    key = key_of_expert[flat.clamp(0, num_experts - 1)]
    key = torch.where((flat >= 0) & (flat < num_experts), key, torch.full_like(key, -1))
    counts_by_key, send_order, pos = route_plan(key, num_experts)
    counts = counts_by_key[key_of_expert]                                 # by global expert
    counts_flat = torch.empty(world * num_experts, dtype=counts.dtype, device=dev)
    dist.all_gather_into_tensor(counts_flat, counts.contiguous(), group=group)
    by_dest = counts_flat.view(world, world, e_loc).permute(1, 2, 0).contiguous()       # [d, l, s]
    flat_blocks = by_dest.view(world, e_loc * world)
    starts = (flat_blocks.cumsum(1) - flat_blocks).view(world, e_loc, world)            # [d, l, s]
    dst_block_start = starts[:, :, me].reshape(num_experts)
    size_per_group = by_dest[me].sum(-1).to(torch.int64).contiguous()     # [e_loc]
    # ---- the one host synchronisation: every rank's per-expert counts (world x num_experts integers);
    # all offsets the host needs follow from them
    ca = counts_flat.cpu().view(world, world, e_loc).numpy()              # [s, d, l]
    host = _host_tables(ca, world, me, e_loc, num_experts, bounds, capacity_rows, key_of_expert_h, expert_of_key)
    send_offsets = host["send_offsets"]
    send_start_by_key = counts_by_key.cumsum(0) - counts_by_key
    valid = send_order[:send_offsets[-1]]
    key_sorted = key[valid]
    e_sorted = flat[valid]
    idx = torch.arange(valid.numel(), device=dev)
    dst_rank = (e_sorted // e_loc).to(torch.int32)
    dst_row = dst_block_start[e_sorted] + (idx - send_start_by_key[key_sorted])
    return PeerChunkPlan(num_tokens=t, top_k=k, bounds=list(bounds), token_of_pair=(valid // k).contiguous(),
                         dst_rank=dst_rank.contiguous(), dst_row=dst_row.contiguous(), pos=pos,
                         size_per_group=size_per_group, **host)


def _host_tables(ca, world, me, e_loc, num_experts, bounds, capacity_rows, key_of_expert_h, expert_of_key) -> dict:
    """Everything the host needs, from every rank's per-expert pair counts ``ca`` [s, d, l] (numpy)."""
    totals = ca.sum(axis=(0, 2))                                          # rows every rank receives
    if int(totals.max()) > capacity_rows:
        raise RuntimeError(f"a rank would receive {int(totals.max())} rows, more than the exchange buffers hold "
                           f"({capacity_rows}); raise capacity_factor")
    blk_count = ca[:, me, :].T.copy()                                     # [l, s] rows of each block here
    blk_start = (blk_count.reshape(-1).cumsum() - blk_count.reshape(-1)).reshape(e_loc, world)
    rows_per_expert = blk_count.sum(axis=1)
    recv_offsets = [int(rows_per_expert[:bb].sum()) for bb in bounds]
    # send order of rank s: its counts in key order; where its pairs for expert (me, l) start
    cbk = ca.reshape(world, num_experts)[:, expert_of_key]               # [s, key]
    send_start = cbk.cumsum(axis=1) - cbk                                 # [s, key]
    ret_row0 = send_start[:, key_of_expert_h[me * e_loc:(me + 1) * e_loc]].T.copy()   # [l, s]
    my_cbk = cbk[me]
    send_offsets = [int(my_cbk[:world * bb].sum()) for bb in bounds]
    # the sender's view of the same blocks: its pairs for expert (d, l) are consecutive in its send
    # order and land as block (l, me) of rank d's [expert][source] layout
    snd_count = ca[me].copy()                                             # [d, l]
    snd_src0 = send_start[me][key_of_expert_h].reshape(world, e_loc).copy()
    per_dest = ca.transpose(1, 2, 0).reshape(world, e_loc * world)        # [d, (l, s)]
    snd_dst0 = (per_dest.cumsum(axis=1) - per_dest).reshape(world, e_loc, world)[:, :, me].copy()
    return dict(send_offsets=send_offsets, recv_offsets=recv_offsets, blk_count=blk_count, blk_start=blk_start,
                ret_row0=ret_row0, snd_count=snd_count, snd_src0=snd_src0, snd_dst0=snd_dst0)


def _make_peer_chunk_plan_cuda(flat, t, k, num_experts, group, capacity_rows, bounds, key_of_expert_h, expert_of_key,
                               key_of_expert, expert_of_key_dev) -> PeerChunkPlan:
    """The same plan with the library's kernels: a counting sort on the permuted expert ids, the
    all-gather of the int32 counts, one layout kernel and one per-pair kernel - instead of some
    thirty small tensor operations."""
    world, me = dist.get_world_size(group), dist.get_rank(group)
    e_loc = num_experts // world
    dev = flat.device
    n = flat.numel()
    lib = _lib.load()
    flat = flat.contiguous()
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    cursor = torch.empty(num_experts, dtype=torch.int32, device=dev)
    order = torch.empty(n, dtype=torch.int64, device=dev)
    pos = torch.empty(n, dtype=torch.int64, device=dev)
    counts_all = torch.empty(world * num_experts, dtype=torch.int32, device=dev)
    scratch = torch.empty(2 * num_experts + e_loc, dtype=torch.int64, device=dev)
    token_of_pair = torch.empty(n, dtype=torch.int64, device=dev)
    dst_rank = torch.empty(n, dtype=torch.int32, device=dev)
    dst_row = torch.empty(n, dtype=torch.int64, device=dev)
    stream = _lib.stream_ptr(dev)
    with torch.cuda.device(dev):
        rc = lib.b200moe_route_plan_mapped(flat.data_ptr(), n, num_experts, key_of_expert.data_ptr(), counts.data_ptr(),
                                           cursor.data_ptr(), order.data_ptr(), pos.data_ptr(), stream)
        _lib.check(rc, "b200moe_route_plan_mapped")
        dist.all_gather_into_tensor(counts_all, counts, group=group)       # [s, key]
        size_per_group = scratch[2 * num_experts:]
        rc = lib.b200moe_peer_plan(counts_all.data_ptr(), expert_of_key_dev.data_ptr(), key_of_expert.data_ptr(), world, me,
                                   num_experts, order.data_ptr(), flat.data_ptr(), n, k, scratch.data_ptr(),
                                   scratch[num_experts:].data_ptr(), size_per_group.data_ptr(), token_of_pair.data_ptr(),
                                   dst_rank.data_ptr(), dst_row.data_ptr(), stream)
        _lib.check(rc, "b200moe_peer_plan")
    # ---- the one host synchronisation (world x num_experts int32); by global expert for the host tables
    ca = counts_all.cpu().view(world, num_experts).numpy()[:, key_of_expert_h].reshape(world, world, e_loc)
    host = _host_tables(ca, world, me, e_loc, num_experts, bounds, capacity_rows, key_of_expert_h, expert_of_key)
    return PeerChunkPlan(num_tokens=t, top_k=k, bounds=list(bounds), token_of_pair=token_of_pair, dst_rank=dst_rank,
                         dst_row=dst_row, pos=pos, size_per_group=size_per_group, **host)


def return_blocks_by_copy(ybuf: PeerBuffer, ret: PeerBuffer, plan: PeerChunkPlan, l_lo: int, l_hi: int,
                          streams=None, after=None) -> None:
    """Results of local experts [l_lo, l_hi) back to their token owners by copy engine: block
    (expert l, source rank s) is contiguous here ([expert][source] layout) and contiguous in s's
    return buffer (s sent those pairs consecutively), so each block is one device-to-device copy
    - over NVLink for the other ranks - and no SM is involved.  ``streams`` (torch streams)
    spreads the copies over several queues, destination rank d on stream d % len(streams), each
    waiting for the event ``after`` first: one queue keeps one copy engine busy, which moves
    ~270 GB/s, a third of what the links carry; without ``streams`` everything goes to the
    current stream."""
    row_bytes = ybuf.local.shape[1] * ybuf.local.element_size()
    assert row_bytes == ret.local.shape[1] * ret.local.element_size()
    n_q = len(streams) if streams else 1
    queues = [([], [], []) for _ in range(n_q)]
    own = ybuf.local.data_ptr()
    for l in range(l_lo, l_hi):
        for s_rank in range(ybuf.world):
            n = int(plan.blk_count[l, s_rank])
            if n:
                assert int(plan.ret_row0[l, s_rank]) + n <= ret.capacity
                dsts, srcs, sizes = queues[s_rank % n_q]
                dsts.append(ret.bases[s_rank] + int(plan.ret_row0[l, s_rank]) * row_bytes)
                srcs.append(own + int(plan.blk_start[l, s_rank]) * row_bytes)
                sizes.append(n * row_bytes)
    lib = _lib.load()
    dev = ybuf.local.device
    for q, (dsts, srcs, sizes) in enumerate(queues):
        stream = streams[q] if streams else torch.cuda.current_stream(dev)
        if after is not None:
            stream.wait_event(after)
        if not dsts:
            continue
        m = len(dsts)
        with torch.cuda.device(dev):
            rc = lib.b200ipc_copy_many_async(m, (ctypes.c_void_p * m)(*dsts), (ctypes.c_void_p * m)(*srcs),
                                             (ctypes.c_int64 * m)(*sizes), stream.cuda_stream)
        _lib.check(rc, "b200ipc_copy_many_async")


def gather_send_rows(x8: torch.Tensor, xs: torch.Tensor, plan: PeerChunkPlan, lo: int, hi: int,
                     send8: torch.Tensor, sends: torch.Tensor) -> None:
    """send8[i], sends[i] = the quantised row and the scales of pair i's token, for the pairs [lo, hi) of
    the send order: the local half of a dispatch by copy engine (two gather kernels, all of HBM's
    bandwidth, nothing crosses NVLink)."""
    if hi <= lo:
        return
    src = x8.view(torch.uint8) if x8.dtype != torch.uint8 else x8
    lib = _lib.load()
    idx = plan.token_of_pair[lo:hi]
    with torch.cuda.device(src.device):
        stream = _lib.stream_ptr(src.device)
        rc = lib.b200moe_gather_rows(src.data_ptr(), idx.data_ptr(), send8[lo:hi].data_ptr(), hi - lo, src.shape[1],
                                     src.shape[0], stream)
        _lib.check(rc, "b200moe_gather_rows")
        rc = lib.b200moe_gather_rows(xs.data_ptr(), idx.data_ptr(), sends[lo:hi].data_ptr(), hi - lo, xs.shape[1] * 4,
                                     xs.shape[0], stream)
        _lib.check(rc, "b200moe_gather_rows")


def dispatch_blocks_by_copy(send8: torch.Tensor, sends: torch.Tensor, rows8: PeerBuffer, scales: PeerBuffer,
                            plan: PeerChunkPlan, l_lo: int, l_hi: int) -> None:
    """The gathered rows of local experts [l_lo, l_hi) of every rank to their owners by copy
    engine: this rank's pairs for expert (d, l) are consecutive in its send order and form block
    (l, this rank) of rank d's [expert][source] buffers, so every block is one device-to-device
    copy of the rows and one of the scales on the current stream; no SM is involved."""
    row_bytes, scale_bytes = send8.shape[1], sends.shape[1] * 4
    assert send8.dtype == torch.uint8 and sends.dtype == torch.float32 and send8.is_contiguous() and sends.is_contiguous()
    assert rows8.local.shape[1] == row_bytes and scales.local.shape[1] * 4 == scale_bytes
    dsts, srcs, sizes = [], [], []
    own8, owns = send8.data_ptr(), sends.data_ptr()
    for d in range(rows8.world):
        for l in range(l_lo, l_hi):
            n = int(plan.snd_count[d, l])
            if n:
                s0, d0 = int(plan.snd_src0[d, l]), int(plan.snd_dst0[d, l])
                assert s0 + n <= send8.shape[0] and d0 + n <= rows8.capacity
                dsts += [rows8.bases[d] + d0 * row_bytes, scales.bases[d] + d0 * scale_bytes]
                srcs += [own8 + s0 * row_bytes, owns + s0 * scale_bytes]
                sizes += [n * row_bytes, n * scale_bytes]
    if not dsts:
        return
    m = len(dsts)
    with torch.cuda.device(send8.device):
        rc = _lib.load().b200ipc_copy_many_async(m, (ctypes.c_void_p * m)(*dsts), (ctypes.c_void_p * m)(*srcs),
                                                 (ctypes.c_int64 * m)(*sizes), _lib.stream_ptr(send8.device))
    _lib.check(rc, "b200ipc_copy_many_async")


def dispatch_quant_range(x: torch.Tensor, plan: PeerChunkPlan, lo: int, hi: int, rows8: PeerBuffer,
                         scales: PeerBuffer, meta: PeerBuffer, blocks: int = 0) -> None:
    """Pairs [lo, hi) of the send order: quantise each pair's token row of ``x`` (bf16 / fp16
    [T, H]) 1x128 and store the e4m3 row, its scales and the pair's return address at the pair's
    row of the owning rank's three buffers (one kernel; ``blocks`` > 0 = that many large blocks,
    for running beside a GEMM)."""
    assert x.is_cuda and x.is_contiguous() and x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16)
    hidden = x.shape[1]
    assert rows8.local.shape[1] * rows8.local.element_size() == hidden
    assert scales.local.dtype == torch.float32 and scales.local.shape[1] == hidden // 128
    assert meta.local.dtype == torch.int64 and meta.local.shape[1] == 2
    assert rows8.capacity == scales.capacity == meta.capacity
    with torch.cuda.device(x.device):
        rc = _lib.load().b200moe_dispatch_quant_rows_multi(
            x.data_ptr(), plan.token_of_pair.data_ptr(), rows8.bases, scales.bases, meta.bases, plan.dst_rank.data_ptr(),
            plan.dst_row.data_ptr(), lo, hi - lo, x.shape[0], hidden, 0 if x.dtype == torch.bfloat16 else 1, rows8.world,
            rows8.capacity, rows8.rank, int(blocks), _lib.stream_ptr(x.device))
    _lib.check(rc, "b200moe_dispatch_quant_rows_multi")


def dispatch_range(x8: torch.Tensor, xs: torch.Tensor, plan: PeerChunkPlan, lo: int, hi: int, rows8: PeerBuffer,
                   scales: PeerBuffer, meta: PeerBuffer, blocks: int = 0) -> None:
    """Pairs [lo, hi) of the send order, rows already quantised (``x8`` fp8 [T, H], ``xs`` fp32
    [T, H/128]): copy each pair's row, scales and return address to the owning rank's buffers."""
    src = x8.view(torch.uint8) if x8.dtype != torch.uint8 else x8
    assert src.is_cuda and src.is_contiguous() and xs.is_contiguous() and xs.dtype == torch.float32
    hidden = src.shape[1]
    assert rows8.local.shape[1] == hidden and scales.local.shape[1] == hidden // 128 == xs.shape[1]
    assert meta.local.dtype == torch.int64 and meta.local.shape[1] == 2
    assert rows8.capacity == scales.capacity == meta.capacity
    with torch.cuda.device(src.device):
        rc = _lib.load().b200moe_dispatch_rows_multi(
            src.data_ptr(), xs.data_ptr(), plan.token_of_pair.data_ptr(), rows8.bases, scales.bases, meta.bases,
            plan.dst_rank.data_ptr(), plan.dst_row.data_ptr(), lo, hi - lo, src.shape[0], hidden, rows8.world,
            rows8.capacity, rows8.rank, int(blocks), _lib.stream_ptr(src.device))
    _lib.check(rc, "b200moe_dispatch_rows_multi")


def return_rows(src: torch.Tensor, meta: torch.Tensor, ret: PeerBuffer, blocks: int = 0) -> None:
    """ret[meta[r, 1]][meta[r, 0]] = src[r] for every row of ``src`` (this rank's results of a
    chunk) - ``meta`` holds the return addresses that arrived beside the rows."""
    assert src.is_contiguous() and meta.is_contiguous() and meta.dtype == torch.int64 and meta.shape == (src.shape[0], 2)
    row_bytes = src.shape[1] * src.element_size()
    assert row_bytes == ret.local.shape[1] * ret.local.element_size()
    with torch.cuda.device(src.device):
        rc = _lib.load().b200moe_return_rows_multi(src.data_ptr(), meta.data_ptr(), ret.bases, src.shape[0], row_bytes,
                                                   ret.world, ret.capacity, int(blocks), _lib.stream_ptr(src.device))
    _lib.check(rc, "b200moe_return_rows_multi")


def scatter_range(src: torch.Tensor, src_idx: torch.Tensor, dst_rank: torch.Tensor, dst_row: torch.Tensor,
                  buf: PeerBuffer, blocks: int = 0) -> None:
    """buf[dst_rank[i]][dst_row[i]] = src[src_idx[i]] for the given index vectors (contiguous tensors
    that the caller keeps alive until the stream has run the kernel)."""
    src2 = src.view(torch.uint8) if src.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else src
    assert src2.is_contiguous() and src_idx.is_contiguous() and dst_rank.is_contiguous() and dst_row.is_contiguous()
    row_bytes = src2.shape[1] * src2.element_size()
    assert row_bytes == buf.local.shape[1] * buf.local.element_size()
    with torch.cuda.device(src2.device):
        rc = _lib.load().b200moe_scatter_rows_multi(src2.data_ptr(), src_idx.data_ptr(), buf.bases, dst_rank.data_ptr(),
                                                    dst_row.data_ptr(), src_idx.numel(), row_bytes, buf.world,
                                                    buf.capacity, src2.shape[0], int(blocks),
                                                    _lib.stream_ptr(src2.device))
    _lib.check(rc, "b200moe_scatter_rows_multi")
