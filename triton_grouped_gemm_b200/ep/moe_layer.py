"""Block-scaled FP8 MoE feed-forward layer with expert parallelism, on the B200 kernels.

Per rank: quantise local tokens 1x128 -> dispatch fp8 rows + scales to the expert owners
(all-to-all) -> gate+up grouped GEMM (fp8, block scaled) -> SwiGLU fused with 1x128
re-quantisation -> down grouped GEMM -> combine (all-to-all back, router-weighted sum).
Weights are quantised 128x128 once at construction.  A decode variant runs the two GEMMs on
the masked layout ([local experts, m_max] slots, ``masked_m`` valid rows each).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..gemm.FP8.m_grouped_gemm_block_scaled import (interleave_gate_up, m_grouped_fp8_block_scaled,
                                                    m_grouped_fp8_block_scaled_masked,
                                                    m_grouped_fp8_block_scaled_swiglu)
from ..quant.per_block_cast import per_block_cast_to_fp8, per_token_cast_to_fp8, swiglu_per_token_cast_to_fp8
from .dispatch import combine, dispatch, dispatch_chunk_async, make_chunked_plan, make_plan, quant_permute_rows


class Fp8MoELayer:
    def __init__(self, w13: torch.Tensor, w2: torch.Tensor, num_experts: int,
                 group: Optional[dist.ProcessGroup] = None, chunks: int = 4, comm_sms: Optional[int] = None,
                 transport: str = "nccl", capacity_factor: float = 1.5, tokens_per_rank: int = 0, top_k: int = 0,
                 quantise_on_dispatch: bool = False, return_path: str = "copy", taper: bool = False,
                 dispatch_path: str = "kernel", ret_streams: int = 2):
        """w13 [E_local, 2*I, H] (gate rows then up rows), w2 [E_local, H, I], bf16, this rank's experts.
        With more than one rank the expert GEMMs consume rows in the order the all-to-all delivers
        them (every [source rank][expert] block is a row group of its own, mapped to its expert's
        weights), so nothing is permuted on the expert side.  ``chunks`` > 1 pipelines the step
        over groups of local experts: the all-to-alls of neighbouring chunks run beside the expert
        GEMMs, which then leave ``comm_sms`` SMs to the collective's kernels.
        ``transport="p2p"`` replaces the all-to-alls by kernels that store / load rows in the
        other ranks' memory directly (``ep/p2p.py``); it needs ``tokens_per_rank`` and ``top_k`` to
        size its buffers: ``capacity_factor`` x the mean number of rows a rank receives.  There the
        received rows are laid out [local expert][source rank], one row group per expert, and
        ``chunks`` (any number up to the local expert count) splits the experts into nearly equal
        runs.  ``quantise_on_dispatch`` (pipelined p2p only) lets the dispatch kernel quantise each
        pair's bf16 token row itself instead of quantising every token once beforehand: same bytes,
        no fp8 copy of the activations in HBM, but a token's row is quantised once per expert it
        goes to, which costs more than it saves when the mover runs on the few SMs beside a GEMM.
        ``return_path`` (pipelined p2p only): "copy" sends every (expert, source rank) block of
        results home with one copy-engine transfer - contiguous on both sides, so the way back
        occupies no SM and the GEMMs keep all but the dispatch movers' SMs; "kernel" uses the
        return-address mover kernel instead.  ``dispatch_path`` (pipelined p2p only): "kernel" (default) moves the
        rows to their experts with the mover kernels on ``comm_sms`` SMs (12 by default) beside the
        GEMMs; "copy" gathers every chunk's rows into send order locally and ships each
        (destination, expert) block with copy-engine transfers too, so that no mover kernel runs beside
        the GEMMs and they keep every SM but ``comm_sms`` (then 2 by default, for the one-word flag
        reductions).  It needs the copy return path, rows quantised beforehand and hidden % 512 == 0
        (else "kernel" is used), and measured slower on two GPUs: the copy engines serve dispatch and
        return at once and a chunk's dispatch stretches from 0.5 to 2.5 ms.  ``taper``: a first and a last run of
        experts about half as long as the others.  ``ret_streams``: stream queues the copy-engine
        return is spread over (by destination rank); one queue keeps one copy engine busy, and at 8
        ranks a single engine (~270 GB/s) cannot keep up with the GEMMs.
        Call ``close()`` on every rank when done with a p2p layer."""
        assert w13.dim() == 3 and w2.dim() == 3 and w13.shape[0] == w2.shape[0]
        self.group = group
        self.num_experts = num_experts
        self.e_local, two_i, self.hidden = w13.shape
        self.inter = two_i // 2
        assert w2.shape == (self.e_local, self.hidden, self.inter)
        self.w13 = per_block_cast_to_fp8(w13.contiguous())
        self.w2 = per_block_cast_to_fp8(w2.contiguous())
        # The decode step (few rows per expert, bound by streaming the weights) uses the gate+up GEMM
        # with SwiGLU and the re-quantisation in its epilogue: 0.70 -> 0.67 ms.  That form needs the
        # two halves interleaved in 128-row blocks - a second quantised copy of w13; for the large
        # prefill / training step it measured slower (the promotion warps that would do the
        # activation already bound the kernel: 10.4 ms against 9.0 + 1.05 ms), so forward() keeps
        # the product and the separate SwiGLU quantiser.
        self.fused_swiglu = self.inter % 128 == 0
        self._w13_interleaved = None   # built by the first decode()
        world = 1 if group is None else dist.get_world_size(group)
        self.world = world
        assert transport in ("nccl", "p2p") and dispatch_path in ("copy", "kernel")
        self.transport = transport if world > 1 else "nccl"
        if self.transport == "nccl":
            while chunks > 1 and self.e_local % chunks:
                chunks -= 1
        self.chunks = max(1, min(chunks, self.e_local)) if world > 1 else 1
        self._peer_buffers = []
        self.quantise_on_dispatch = bool(quantise_on_dispatch)
        assert return_path in ("copy", "kernel")
        self.return_path = return_path
        self.dispatch_path = dispatch_path if (return_path == "copy" and not quantise_on_dispatch
                                               and self.hidden % 512 == 0) else "kernel"
        movers = not (self.transport == "p2p" and self.chunks > 1 and self.dispatch_path == "copy")
        self.comm_sms = comm_sms if comm_sms is not None else (12 if movers else 2)
        self.trace = False
        self._marks = None
        if self.transport == "p2p":
            from .p2p import PeerBuffer, chunk_bounds

            assert tokens_per_rank > 0 and top_k > 0, "the p2p transport sizes its buffers from tokens_per_rank and top_k"
            assert self.hidden % 128 == 0, "the p2p transport moves 1x128-quantised rows: hidden must be a multiple of 128"
            # the one-shot form moves the scales with the generic 16-byte-vector scatter: 4 * hidden / 128 bytes per row
            assert self.chunks > 1 or self.hidden % 512 == 0, \
                "transport='p2p' with chunks=1 needs hidden % 512 == 0 (scale rows of a multiple of 16 bytes); use chunks > 1"
            cap = (int(tokens_per_rank * top_k * capacity_factor) + 255) // 256 * 256
            dev = w13.device
            self.bounds = chunk_bounds(self.e_local, self.chunks, taper)
            self.chunks = len(self.bounds) - 1
            self.recv8 = PeerBuffer(cap, self.hidden, torch.uint8, dev, group)
            self.recvs = PeerBuffer(cap, self.hidden // 128, torch.float32, dev, group)
            self.ybuf = PeerBuffer(cap, self.hidden, torch.bfloat16, dev, group)
            self._peer_buffers = [self.recv8, self.recvs, self.ybuf]
            self._flag = torch.zeros(1, dtype=torch.int32, device=dev)
            if self.chunks > 1:
                # pipelined form: results are pushed back into the token owner's buffer chunk by chunk
                self.meta = PeerBuffer(cap, 2, torch.int64, dev, group)
                self.ret = PeerBuffer(tokens_per_rank * top_k, self.hidden, torch.bfloat16, dev, group)
                self._peer_buffers += [self.meta, self.ret]
                self._side = (torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
                # further queues for the copy-engine return: one queue feeds one copy engine (~270 GB/s)
                self._ret_extra = [torch.cuda.Stream(device=dev) for _ in range(max(0, min(ret_streams, world) - 1))]
                if self.dispatch_path == "copy":
                    # this rank's rows in send order, the source of the copy-engine dispatch
                    self._send8 = torch.empty((tokens_per_rank * top_k, self.hidden), dtype=torch.uint8, device=dev)
                    self._sends = torch.empty((tokens_per_rank * top_k, self.hidden // 128), dtype=torch.float32, device=dev)

    @property
    def w13_interleaved(self):
        """Gate and up rows interleaved in 128-row blocks, quantised: the weight layout of the
        gate+up GEMM with the SwiGLU epilogue.  Only decode() needs it, so this second quantised
        copy of w13 is built on first use."""
        if self._w13_interleaved is None and self.fused_swiglu:
            # 128x128 quantisation commutes with the interleave (whole scale blocks move): permute the
            # quantised bytes in 128-row blocks and the scale matrix in single rows
            q, sc = self.w13
            e, two_i, _ = q.shape
            sc_il = sc.reshape(e, 2, two_i // 256, sc.shape[-1]).transpose(1, 2).reshape(e, two_i // 128, -1)
            self._w13_interleaved = (interleave_gate_up(q.view(torch.uint8)).view(q.dtype), sc_il.contiguous())
        return self._w13_interleaved

    def close(self) -> None:
        """Releases the peer-memory buffers of transport="p2p".  Collective: every rank calls it,
        after its last forward().  The last step of forward() reads or writes the other ranks'
        buffers, and nothing after it orders those accesses against a rank that goes on to free
        its memory; so this waits for the device, meets the other ranks at a barrier, and only then
        unmaps and frees (a rank must not leave or free between its last forward() and that
        barrier).  Safe to call twice; a layer with another transport has nothing to release."""
        if not self._peer_buffers:
            return
        torch.cuda.synchronize(self.recv8.local.device)
        dist.barrier(group=self.group)
        for buf in self._peer_buffers:
            buf.close(self.group)
        self._peer_buffers = []

    def experts(self, x8: torch.Tensor, xs: torch.Tensor, size_per_group: torch.Tensor,
                group_to_expert: Optional[torch.Tensor] = None, num_sms: int = -1,
                out: Optional[torch.Tensor] = None, first_expert: int = 0) -> torch.Tensor:
        """Rows grouped by local expert: [R, H] fp8 + scales -> [R, H] bf16.  With
        ``group_to_expert`` (int32) the row groups are arbitrary blocks, block i using the
        weights of local expert ``group_to_expert[i]``; without it, group i uses local expert
        ``first_expert + i`` (``size_per_group`` may cover a run of the experts only)."""
        w13, w2 = self.w13, self.w2
        if group_to_expert is None and (first_expert or size_per_group.numel() != self.e_local):
            hi = first_expert + size_per_group.numel()
            w13 = (w13[0][first_expert:hi], w13[1][first_expert:hi])
            w2 = (w2[0][first_expert:hi], w2[1][first_expert:hi])
        h = m_grouped_fp8_block_scaled((x8, xs), w13, size_per_group, num_sms=num_sms, group_to_b=group_to_expert)
        a8, a_s = swiglu_per_token_cast_to_fp8(h)
        return m_grouped_fp8_block_scaled((a8, a_s), w2, size_per_group, num_sms=num_sms,
                                          group_to_b=group_to_expert, out=out)

    def _forward_p2p(self, x8, xs, topk_idx, topk_weight) -> torch.Tensor:
        """All ranks: scatter rows into their owners' buffers | barrier | GEMMs on the local
        buffers | barrier | weighted sum reading the owners' results."""
        from .p2p import combine_rows, make_peer_plan, scatter_rows

        plan = make_peer_plan(topk_idx, self.num_experts, self.group, self.recv8.capacity)
        scatter_rows(plan, x8, self.recv8)
        scatter_rows(plan, xs, self.recvs)
        dist.all_reduce(self._flag, group=self.group)       # every rank's rows have landed everywhere
        r = plan.rows_here
        self.last_rows = (r, plan.size_per_group)   # rows received this step and their split over the experts
        self.experts(self.recv8.local[:r].view(torch.float8_e4m3fn), self.recvs.local[:r], plan.size_per_group,
                     out=self.ybuf.local[:r])
        dist.all_reduce(self._flag, group=self.group)       # every rank's results are written
        return combine_rows(plan, self.ybuf, topk_weight)

    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weight: torch.Tensor) -> torch.Tensor:
        """x [T, H] bf16, topk_idx/topk_weight [T, k] -> [T, H] bf16."""
        if self.transport == "p2p" and self.chunks > 1:
            return self._forward_p2p_pipelined(x.contiguous(), topk_idx, topk_weight)  # quantises while it dispatches
        x = x.contiguous()
        if self.world == 1:
            plan = make_plan(topk_idx, self.num_experts, self.group)
            if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and self.hidden % 128 == 0 and self.hidden <= 8192:
                # one rank: quantise every token once and write it straight to its k expert-major rows
                r8, rs = quant_permute_rows(x, plan.pos, plan.top_k)
            else:
                x8, xs = per_token_cast_to_fp8(x)
                r8, rs = dispatch(plan, x8, self.group).contiguous(), dispatch(plan, xs, self.group).contiguous()
            y = self.experts(r8, rs, plan.size_per_group)
            return combine(plan, y, topk_weight, self.group)
        x8, xs = per_token_cast_to_fp8(x)
        if self.transport == "p2p":
            return self._forward_p2p(x8, xs, topk_idx, topk_weight)
        return self._forward_pipelined(x8, xs, topk_idx, topk_weight)

    def _forward_pipelined(self, x8, xs, topk_idx, topk_weight) -> torch.Tensor:
        """More than one rank.  Chunk c's GEMMs run while chunk c+1 is being dispatched and chunk
        c-1 combined (the collectives are asynchronous on the process group's own stream)."""
        from .. import _lib

        plan = make_chunked_plan(topk_idx, self.num_experts, self.group, self.chunks, with_permutation=False)
        sms = _lib.load().b200gemm_sm_count()
        gemm_sms = sms - self.comm_sms if (self.chunks > 1 and 0 < self.comm_sms < sms - 2) else -1
        total_pairs = plan.send_order.numel()
        ret = torch.empty((total_pairs, self.hidden), dtype=torch.bfloat16, device=x8.device)
        pending = []
        nxt = dispatch_chunk_async(plan, 0, (x8, xs), self.group)
        for c in range(self.chunks):
            recvs, works, keep = nxt
            nxt = dispatch_chunk_async(plan, c + 1, (x8, xs), self.group) if c + 1 < self.chunks else None
            for w in works:
                w.wait()
            # rows stay in arrival order: [source rank][expert of the chunk] blocks
            y = self.experts(recvs[0].view(torch.float8_e4m3fn), recvs[1], plan.block_sizes[c],
                             group_to_expert=plan.block_expert[c], num_sms=gemm_sms)
            lo, hi = plan.send_offsets[c], plan.send_offsets[c + 1]
            pending.append((dist.all_to_all_single(ret[lo:hi], y, output_split_sizes=plan.send_splits[c],
                                                   input_split_sizes=plan.recv_splits[c], group=self.group,
                                                   async_op=True), y, keep, recvs))
        for w, *_ in pending:
            w.wait()
        pos = plan.pos  # position of pair (t, k) among the returned rows (send order is chunk-major)
        out = torch.empty((plan.num_tokens, self.hidden), dtype=torch.bfloat16, device=x8.device)
        w32 = topk_weight.reshape(-1).to(torch.float32).contiguous()
        with torch.cuda.device(x8.device):
            rc = _lib.load().b200moe_combine_topk(ret.data_ptr(), pos.data_ptr(), w32.data_ptr(), out.data_ptr(),
                                                  plan.num_tokens, plan.top_k, self.hidden, ret.shape[0],
                                                  _lib.stream_ptr(x8.device))
        _lib.check(rc, "b200moe_combine_topk")
        return out

    def _forward_p2p_pipelined(self, x, topk_idx, topk_weight) -> torch.Tensor:
        """Peer memory in both directions, beside the GEMMs.  A dispatch stream sends chunk after
        chunk: one kernel per chunk stores each pair's fp8 row, its scales and the pair's return
        address into the owner's buffers (rows quantised once up front, or - with
        ``quantise_on_dispatch`` - by that same kernel from the bf16 rows).  The main stream runs
        chunk c's GEMMs (one row group per expert) as soon as its rows have landed everywhere; a
        return stream sends chunk c's results to the token owners' buffers: one copy-engine
        transfer per (expert, source rank) block, or the return-address mover kernel.  Movers that
        run beside a GEMM are a few large blocks on the SMs the GEMMs leave free; the first
        dispatch (and the last return kernel) use the whole GPU.  A local weighted sum
        finishes the step.  With ``self.trace`` set, CUDA events bracket every phase on its stream
        (``phase_times()`` reads them)."""
        from .. import _lib
        from .p2p import (dispatch_blocks_by_copy, dispatch_quant_range, dispatch_range, gather_send_rows,
                          make_peer_chunk_plan, return_blocks_by_copy, return_rows)

        lib = _lib.load()
        dev = x.device
        main = torch.cuda.current_stream(dev)
        marks = [] if self.trace else None

        def mark(name, stream):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                marks.append((name, ev))

        mark("start", main)
        if not self.quantise_on_dispatch:
            x8, xs = per_token_cast_to_fp8(x)   # queued first: runs while the host waits for the plan's counts
        plan = make_peer_chunk_plan(topk_idx, self.num_experts, self.group, self.recv8.capacity, self.bounds)
        assert plan.pos.numel() <= self.ret.capacity, "more (token, k) pairs than the return buffer holds"
        self.last_rows = (plan.recv_offsets[-1], plan.size_per_group)
        mark("plan_done", main)
        chunks = plan.chunks
        sms = lib.b200gemm_sm_count()
        gemm_sms = sms - self.comm_sms if 0 < self.comm_sms < sms - 2 else -1
        s_disp, s_ret = self._side
        ready = torch.cuda.Event()
        ready.record(main)
        landed = [torch.cuda.Event() for _ in range(chunks)]
        computed = [torch.cuda.Event() for _ in range(chunks)]
        background = max(self.comm_sms, 1)
        with torch.cuda.stream(s_disp):
            s_disp.wait_event(ready)
            for c in range(chunks):
                lo, hi = plan.send_offsets[c], plan.send_offsets[c + 1]
                blocks = 0 if c == 0 else background
                mark(f"dispatch{c}>", s_disp)
                if self.dispatch_path == "copy":
                    # chunk 0's rows are gathered alone so that its copies start at once; the other
                    # chunks' rows in one go on the (still idle) return stream, while chunk 0 is on
                    # the wire and before the first GEMM starts
                    if c == 0:
                        gather_send_rows(x8, xs, plan, lo, hi, self._send8, self._sends)
                        gathered0 = torch.cuda.Event()
                        gathered0.record(s_disp)
                        with torch.cuda.stream(s_ret):
                            s_ret.wait_event(gathered0)
                            gather_send_rows(x8, xs, plan, hi, plan.send_offsets[-1], self._send8, self._sends)
                            gathered = torch.cuda.Event()
                            gathered.record(s_ret)
                    elif c == 1:
                        s_disp.wait_event(gathered)
                    dispatch_blocks_by_copy(self._send8, self._sends, self.recv8, self.recvs, plan,
                                            self.bounds[c], self.bounds[c + 1])
                elif self.quantise_on_dispatch:
                    dispatch_quant_range(x, plan, lo, hi, self.recv8, self.recvs, self.meta, blocks=blocks)
                else:
                    dispatch_range(x8, xs, plan, lo, hi, self.recv8, self.recvs, self.meta, blocks=blocks)
                mark(f"dispatch{c}<", s_disp)
                dist.all_reduce(self._flag, group=self.group)      # chunk c has landed on every rank
                landed[c].record(s_disp)
                mark(f"landed{c}", s_disp)
        for c in range(chunks):
            lo, hi = plan.recv_offsets[c], plan.recv_offsets[c + 1]
            main.wait_event(landed[c])
            mark(f"gemm{c}>", main)
            self.experts(self.recv8.local[lo:hi].view(torch.float8_e4m3fn), self.recvs.local[lo:hi],
                         plan.size_per_group[self.bounds[c]:self.bounds[c + 1]], num_sms=gemm_sms,
                         out=self.ybuf.local[lo:hi], first_expert=self.bounds[c])
            mark(f"gemm{c}<", main)
            computed[c].record(main)
            with torch.cuda.stream(s_ret):
                s_ret.wait_event(computed[c])
                mark(f"return{c}>", s_ret)
                if self.return_path == "copy":
                    queues = [s_ret] + self._ret_extra
                    return_blocks_by_copy(self.ybuf, self.ret, plan, self.bounds[c], self.bounds[c + 1],
                                          streams=queues, after=computed[c])
                    for q in self._ret_extra:      # s_ret stands for the whole chunk again
                        joined = torch.cuda.Event()
                        joined.record(q)
                        s_ret.wait_event(joined)
                else:
                    return_rows(self.ybuf.local[lo:hi], self.meta.local[lo:hi], self.ret,
                                blocks=0 if c == chunks - 1 else background)
                mark(f"return{c}<", s_ret)
        with torch.cuda.stream(s_ret):
            dist.all_reduce(self._flag, group=self.group)          # every rank's results have been pushed
            done = torch.cuda.Event()
            done.record(s_ret)
            mark("returned_everywhere", s_ret)
        main.wait_event(done)
        out = torch.empty((plan.num_tokens, self.hidden), dtype=torch.bfloat16, device=dev)
        w32 = topk_weight.reshape(-1).to(torch.float32).contiguous()
        with torch.cuda.device(dev):
            rc = lib.b200moe_combine_topk(self.ret.local.data_ptr(), plan.pos.data_ptr(), w32.data_ptr(), out.data_ptr(),
                                          plan.num_tokens, plan.top_k, self.hidden, self.ret.capacity,
                                          _lib.stream_ptr(dev))
        _lib.check(rc, "b200moe_combine_topk")
        mark("end", main)
        self._marks = marks
        return out

    def phase_times(self):
        """After a pipelined peer-memory step with ``trace`` set: [(phase, ms since the step's
        start)] for every mark, in the order they were recorded (synchronises the device)."""
        if not getattr(self, "_marks", None):
            return []
        torch.cuda.synchronize()
        t0 = self._marks[0][1]
        return [(name, t0.elapsed_time(ev)) for name, ev in self._marks]

    def decode(self, x8: torch.Tensor, xs: torch.Tensor, masked_m: torch.Tensor, m_max: int,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Masked layout: x8 [E_local*m_max, H] fp8 + scales, ``masked_m`` valid rows per expert.
        Rows past ``masked_m[e]`` of each slot are left as they were in ``out`` (zeros if None)."""
        rows = self.e_local * m_max
        assert x8.shape == (rows, self.hidden)
        if self.fused_swiglu:
            a8, a_s = m_grouped_fp8_block_scaled_swiglu((x8, xs), self.w13_interleaved, masked_m, masked_stride=m_max)
        else:
            h = torch.zeros((rows, 2 * self.inter), device=x8.device, dtype=torch.bfloat16)
            m_grouped_fp8_block_scaled_masked((x8, xs), self.w13, h, masked_m, m_max)
            a8, a_s = swiglu_per_token_cast_to_fp8(h)
        if out is None:
            out = torch.zeros((rows, self.hidden), device=x8.device, dtype=torch.bfloat16)
        m_grouped_fp8_block_scaled_masked((a8, a_s), self.w2, out, masked_m, m_max)
        return out


def synthetic_routing(num_tokens: int, num_experts: int, top_k: int, seed: int,
                      device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """Router of the benchmark configuration: logits ~ N(0, 0.5), softmax, top-k (weights
    renormalised over the selected experts)."""
    gen = torch.Generator().manual_seed(seed)
    logits = 0.5 * torch.randn(num_tokens, num_experts, generator=gen)
    p = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(p, top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    return idx.to(device), w.to(device)
