"""Token dispatch / combine for expert parallelism (device-agnostic torch + torch.distributed).

Each rank owns ``experts_per_rank`` consecutive experts.  ``make_plan`` sorts a rank's
(token, k) routing pairs by destination expert, exchanges the per-expert counts, and records
how received rows (ordered by source rank, then expert) map to expert-major order, which is
the row layout the grouped GEMMs consume (``size_per_group`` = rows per local expert).
``dispatch`` moves row payloads (any dtype, e.g. fp8 bytes and their fp32 scales) to the
owning ranks; ``combine`` brings per-row results back and sums the top-k contributions of a
token with the router weights.  The only collectives are all_to_all_single calls; on GPUs the
process group is NCCL, in the CPU tests it is gloo.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    world: int
    experts_per_rank: int
    num_tokens: int
    top_k: int
    send_order: torch.Tensor        # [T*k] indices into the flattened (token, k) pairs, sorted by expert
    send_splits: List[int]          # rows sent to each rank
    recv_splits: List[int]          # rows received from each rank
    recv_to_expert_major: torch.Tensor  # [R] permutation: expert-major row i = received row perm[i]
    size_per_group: torch.Tensor    # [experts_per_rank] rows per local expert (int64, on the data device)
    pos: Optional[torch.Tensor] = None  # [T*k] position of pair (t, k) in send order (send_order^-1)

    @property
    def rows_received(self) -> int:
        return int(sum(self.recv_splits))


def _gather_rows(rows: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """rows[idx] for 2-D rows; on CUDA through the library's gather kernel (no fallback needed on
    CPU tensors: those are the gloo tests of the host logic)."""
    if rows.is_cuda and rows.dim() == 2 and rows.is_contiguous() and (rows.shape[1] * rows.element_size()) % 16 == 0:
        from .. import _lib

        out = torch.empty((idx.numel(), rows.shape[1]), dtype=rows.dtype, device=rows.device)
        idx64 = idx.to(torch.int64).contiguous()
        with torch.cuda.device(rows.device):
            rc = _lib.load().b200moe_gather_rows(rows.data_ptr(), idx64.data_ptr(), out.data_ptr(), idx64.numel(),
                                                 rows.shape[1] * rows.element_size(), rows.shape[0],
                                                 _lib.stream_ptr(rows.device))
        _lib.check(rc, "b200moe_gather_rows")
        return out
    return rows[idx]


def quant_permute_rows(x: torch.Tensor, pos: torch.Tensor, top_k: int):
    """x [T, H] bf16 / fp16 on CUDA, pos [T*k] int64 (row of pair (t, j) in expert-major order, -1 =
    dropped): returns (rows8 [T*k, H] float8_e4m3fn, scales [T*k, H/128] fp32) with
    rows8[pos[t*k+j]], scales[pos[t*k+j]] = the 1x128 quantisation of x[t] - what
    ``per_token_cast_to_fp8`` followed by a gather in send order gives, in one kernel."""
    from .. import _lib

    assert x.is_cuda and x.dim() == 2 and x.is_contiguous() and x.dtype in (torch.bfloat16, torch.float16)
    t, h = x.shape
    assert pos.numel() == t * top_k and pos.dtype == torch.int64 and pos.is_contiguous()
    rows8 = torch.empty((t * top_k, h), dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty((t * top_k, h // 128), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().b200moe_quant_scatter_rows(x.data_ptr(), 0 if x.dtype == torch.bfloat16 else 1, t, h,
                                                    pos.data_ptr(), top_k, rows8.data_ptr(), scales.data_ptr(),
                                                    t * top_k, _lib.stream_ptr(x.device))
    _lib.check(rc, "b200moe_quant_scatter_rows")
    return rows8, scales


def route_plan(keys: torch.Tensor, num_keys: int):
    """Counting sort of ``keys`` (int64, values in [0, num_keys)): returns (counts int64 [num_keys],
    order int64 [n] - indices grouped by key, pos = order^-1).  On CUDA one pass of the library's
    routing-plan kernels (order inside a key's range unspecified); on the host a stable argsort.
    A key outside the range (a dropped token's -1) is counted nowhere and gets pos = -1; the slots
    it leaves at the end of ``order`` hold -1.  The row movers skip negative indices."""
    n = keys.numel()
    if keys.is_cuda and num_keys <= 1024:
        from .. import _lib

        keys = keys.contiguous()
        counts = torch.empty(num_keys, dtype=torch.int32, device=keys.device)
        cursor = torch.empty(num_keys, dtype=torch.int32, device=keys.device)
        order = torch.empty(n, dtype=torch.int64, device=keys.device)
        pos = torch.empty(n, dtype=torch.int64, device=keys.device)
        with torch.cuda.device(keys.device):
            rc = _lib.load().b200moe_route_plan(keys.data_ptr(), n, num_keys, counts.data_ptr(), cursor.data_ptr(),
                                                order.data_ptr(), pos.data_ptr(), _lib.stream_ptr(keys.device))
        _lib.check(rc, "b200moe_route_plan")
        return counts.to(torch.int64), order, pos
    # host tensors (the gloo tests): a stable argsort; keys outside [0, num_keys) are rejected like
    # the kernels do - counted nowhere, pos = -1, their slots at the end of `order` = -1
    ok = (keys >= 0) & (keys < num_keys)
    order = torch.argsort(torch.where(ok, keys, torch.full_like(keys, num_keys)), stable=True)
    n_ok = int(ok.sum())
    pos = torch.full_like(order, -1)
    pos[order[:n_ok]] = torch.arange(n_ok, device=keys.device)
    order = torch.cat([order[:n_ok], order.new_full((n - n_ok,), -1)])
    return torch.bincount(keys[ok], minlength=num_keys), order, pos


def _all_to_all(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, group) -> None:
    if group is None or dist.get_world_size(group) == 1:
        out.copy_(inp)
        return
    dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)


def make_plan(topk_idx: torch.Tensor, num_experts: int, group: Optional[dist.ProcessGroup] = None) -> DispatchPlan:
    """topk_idx [T, k] (global expert ids of this rank's tokens)."""
    world = 1 if group is None else dist.get_world_size(group)
    assert num_experts % world == 0, "experts must divide evenly over the ranks"
    e_loc = num_experts // world
    t, k = topk_idx.shape
    dev = topk_idx.device
    flat = topk_idx.reshape(-1).to(torch.int64)
    counts, send_order, pos = route_plan(flat, num_experts)          # rows per destination expert
    if world == 1:
        # one rank: the send order already is expert-major; nothing to exchange, no host synchronisation
        return DispatchPlan(world=1, experts_per_rank=e_loc, num_tokens=t, top_k=k, send_order=send_order,
                            send_splits=[t * k], recv_splits=[t * k],
                            recv_to_expert_major=torch.arange(t * k, device=dev), size_per_group=counts, pos=pos)
    recv_counts = torch.empty_like(counts)                           # [world * e_loc]: from rank r, expert e
    _all_to_all(recv_counts, counts, None, None, group)
    send_splits = counts.view(world, e_loc).sum(1).tolist()
    recv_matrix = recv_counts.view(world, e_loc)
    recv_splits = recv_matrix.sum(1).tolist()
    # received rows come as [source rank][local expert][rows]; expert-major wants [expert][source][rows]
    blocks = recv_matrix.reshape(-1)                                 # block (r, e) sizes in arrival order
    starts = torch.cumsum(blocks, 0) - blocks
    order = torch.arange(world * e_loc, device=dev).view(world, e_loc).t().reshape(-1)  # (e, r) order
    total = int(sum(recv_splits))
    blk_sizes = blocks[order]
    blk_starts = starts[order]
    out_starts = torch.cumsum(blk_sizes, 0) - blk_sizes
    row_block = torch.repeat_interleave(torch.arange(order.numel(), device=dev), blk_sizes, output_size=total)
    perm = blk_starts[row_block] + (torch.arange(total, device=dev) - out_starts[row_block])
    return DispatchPlan(world=world, experts_per_rank=e_loc, num_tokens=t, top_k=k, send_order=send_order,
                        send_splits=send_splits, recv_splits=recv_splits, recv_to_expert_major=perm,
                        size_per_group=recv_matrix.sum(0).to(torch.int64), pos=pos)


@dataclass
class ChunkedPlan:
    """Routing of one step split into ``chunks`` groups of local experts (chunk c = local experts
    [c*ec, (c+1)*ec) on EVERY rank), so that the exchange of chunk c+1 can run beside the expert
    GEMMs of chunk c.  Rows are sent chunk-major: chunk, destination rank, expert."""
    world: int
    experts_per_rank: int
    chunks: int
    num_tokens: int
    top_k: int
    send_order: torch.Tensor            # [T*k] indices into the flattened (token, k) pairs, chunk-major
    send_offsets: List[int]             # [chunks + 1] row offsets of the chunks in send order
    send_splits: List[List[int]]        # [chunks][world] rows sent to each rank
    recv_splits: List[List[int]]        # [chunks][world] rows received from each rank
    recv_to_expert_major: List[torch.Tensor]  # per chunk: expert-major row i = received row perm[i]
    size_per_group: List[torch.Tensor]  # per chunk: [ec] rows per local expert of the chunk (int64)
    block_sizes: List[torch.Tensor]     # per chunk: [world*ec] rows of each (source rank, expert) block, arrival order
    block_expert: List[torch.Tensor]    # per chunk: [world*ec] local expert (0..e_loc) of each block, int32
    pos: Optional[torch.Tensor] = None  # [T*k] position of pair (t, k) in send order


def make_chunked_plan(topk_idx: torch.Tensor, num_experts: int, group: Optional[dist.ProcessGroup],
                      chunks: int, with_permutation: bool = True) -> ChunkedPlan:
    """Like ``make_plan`` for ``chunks`` expert groups at once; one host synchronisation.
    ``with_permutation=False`` skips the expert-major permutations (callers that feed the
    received blocks to the GEMM as they arrive do not need them)."""
    world = 1 if group is None else dist.get_world_size(group)
    assert num_experts % world == 0, "experts must divide evenly over the ranks"
    e_loc = num_experts // world
    assert e_loc % chunks == 0, "chunks must divide the experts of a rank"
    ec = e_loc // chunks
    t, k = topk_idx.shape
    dev = topk_idx.device
    flat = topk_idx.reshape(-1).to(torch.int64)
    rank_of = flat // e_loc
    local = flat - rank_of * e_loc
    chunk_of = local // ec
    key = chunk_of * (world * ec) + rank_of * ec + (local - chunk_of * ec)
    counts_by_key, send_order, pos = route_plan(key, num_experts)
    # key of expert e = (rank r, chunk c, j): c * (world * ec) + r * ec + j
    e_ids = torch.arange(num_experts, device=dev)
    e_rank, e_local = e_ids // e_loc, e_ids % e_loc
    counts = counts_by_key[(e_local // ec) * (world * ec) + e_rank * ec + e_local % ec]   # [world * e_loc]
    recv_counts = torch.empty_like(counts)                                     # from rank r, local expert e
    _all_to_all(recv_counts, counts, None, None, group)
    send_m = counts.view(world, chunks, ec).sum(-1).t().contiguous()           # [chunks, world]
    recv_3 = recv_counts.view(world, chunks, ec)
    recv_m = recv_3.sum(-1).t().contiguous()                                   # [chunks, world]
    both = torch.stack([send_m, recv_m]).cpu()                                 # the one host sync
    send_splits, recv_splits = both[0].tolist(), both[1].tolist()
    send_offsets = [0]
    for c in range(chunks):
        send_offsets.append(send_offsets[-1] + int(sum(send_splits[c])))
    perms, sizes, block_sizes, block_expert = [], [], [], []
    for c in range(chunks):
        recv_matrix = recv_3[:, c, :]                                          # [world, ec]
        block_sizes.append(recv_matrix.reshape(-1).to(torch.int64).contiguous())
        block_expert.append((torch.arange(ec, device=dev, dtype=torch.int32) + c * ec).repeat(world).contiguous())
        sizes.append(recv_matrix.sum(0).to(torch.int64))
        if not with_permutation:
            perms.append(None)
            continue
        blocks = recv_matrix.reshape(-1)
        starts = torch.cumsum(blocks, 0) - blocks
        order = torch.arange(world * ec, device=dev).view(world, ec).t().reshape(-1)
        total = int(sum(recv_splits[c]))
        blk_sizes = blocks[order]
        blk_starts = starts[order]
        out_starts = torch.cumsum(blk_sizes, 0) - blk_sizes
        row_block = torch.repeat_interleave(torch.arange(order.numel(), device=dev), blk_sizes, output_size=total)
        perms.append(blk_starts[row_block] + (torch.arange(total, device=dev) - out_starts[row_block]))
    return ChunkedPlan(world=world, experts_per_rank=e_loc, chunks=chunks, num_tokens=t, top_k=k,
                       send_order=send_order, send_offsets=send_offsets, send_splits=send_splits,
                       recv_splits=recv_splits, recv_to_expert_major=perms, size_per_group=sizes,
                       block_sizes=block_sizes, block_expert=block_expert, pos=pos)


def dispatch_chunk_async(plan: ChunkedPlan, c: int, payloads, group):
    """Starts the exchange of chunk ``c`` for every tensor of ``payloads`` ([T, ...] per token).
    Returns (received tensors in arrival order, work handles, tensors to keep alive)."""
    lo, hi = plan.send_offsets[c], plan.send_offsets[c + 1]
    token_of_pair = plan.send_order[lo:hi] // plan.top_k
    total = int(sum(plan.recv_splits[c]))
    recvs, works, keep = [], [], []
    for rows in payloads:
        src = rows.view(torch.uint8) if rows.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else rows
        send = _gather_rows(src, token_of_pair)
        recv = torch.empty((total,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        works.append(dist.all_to_all_single(recv, send, output_split_sizes=plan.recv_splits[c],
                                            input_split_sizes=plan.send_splits[c], group=group, async_op=True))
        recvs.append(recv)
        keep.append(send)
    return recvs, works, keep


def dispatch(plan: DispatchPlan, rows: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """rows [T, ...] per token -> [R, ...] rows for this rank's experts, expert-major."""
    token_of_pair = plan.send_order // plan.top_k
    src = rows.view(torch.uint8) if rows.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else rows
    send = _gather_rows(src, token_of_pair)
    if plan.world == 1:
        out = send  # one rank: the send order already is expert-major
    else:
        recv = torch.empty((plan.rows_received,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        _all_to_all(recv, send, plan.recv_splits, plan.send_splits, group)
        out = _gather_rows(recv, plan.recv_to_expert_major)
    return out.view(rows.dtype) if src.dtype != rows.dtype else out


def combine(plan: DispatchPlan, expert_rows: torch.Tensor, topk_weight: torch.Tensor,
            group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """expert_rows [R, H] (expert-major results) -> [T, H]: sum_k weight[t,k] * result(t,k)."""
    if plan.world == 1:
        ret = expert_rows                                             # already in send order
    else:
        inv = torch.empty_like(plan.recv_to_expert_major)
        inv[plan.recv_to_expert_major] = torch.arange(inv.numel(), device=inv.device)
        back = _gather_rows(expert_rows, inv)                         # arrival order again
        ret = torch.empty((plan.send_order.numel(), expert_rows.shape[1]), dtype=expert_rows.dtype,
                          device=expert_rows.device)
        _all_to_all(ret, back, plan.send_splits, plan.recv_splits, group)
    # position of pair (t, k) among the returned rows
    pos = plan.pos
    if pos is None:
        pos = torch.empty_like(plan.send_order)
        pos[plan.send_order] = torch.arange(pos.numel(), device=pos.device)
    if ret.is_cuda and ret.dtype == torch.bfloat16 and ret.shape[1] % 8 == 0:
        from .. import _lib

        out = torch.empty((plan.num_tokens, ret.shape[1]), dtype=ret.dtype, device=ret.device)
        w32 = topk_weight.reshape(-1).to(torch.float32).contiguous()
        with torch.cuda.device(ret.device):
            rc = _lib.load().b200moe_combine_topk(ret.data_ptr(), pos.data_ptr(), w32.data_ptr(), out.data_ptr(),
                                                  plan.num_tokens, plan.top_k, ret.shape[1], ret.shape[0],
                                                  _lib.stream_ptr(ret.device))
        _lib.check(rc, "b200moe_combine_topk")
        return out
    pair_rows = ret[pos]                                              # (token, k) order
    w = topk_weight.reshape(plan.num_tokens, plan.top_k, 1).to(torch.float32)
    return (pair_rows.view(plan.num_tokens, plan.top_k, -1).to(torch.float32) * w).sum(1).to(expert_rows.dtype)
