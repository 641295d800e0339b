"""The FP8 block-scaled MoE layer (quantise -> dispatch -> gate+up -> SwiGLU+quantise -> down ->
combine) on one GPU against the fp32 CPU restatement, plus the fused SwiGLU quantiser and the
masked decode variant.  Tolerance: each GEMM is held to rdiff <= 2e-3 in its own tests; the
layer chains two quantisation steps whose inputs may differ by one bf16 ulp between the GPU
(expf) and the host (vectorised exp), which can flip an e4m3 byte, so the layer is checked
at rdiff <= 5e-3."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.ep.moe_layer import Fp8MoELayer, synthetic_routing
from triton_grouped_gemm_b200.quant.per_block_cast import per_token_cast_to_fp8, swiglu_per_token_cast_to_fp8

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert _lib.device_status() == 0


def test_swiglu_quant_matches_two_step_reference():
    gen = torch.Generator().manual_seed(0)
    h = (torch.randn(300, 512, generator=gen) * 2).bfloat16()
    q, s = swiglu_per_token_cast_to_fp8(h.to(DEV))
    act = (torch.nn.functional.silu(h[:, :256].float()) * h[:, 256:].float()).bfloat16()
    q_ref, s_ref = O.per_token_cast_to_fp8(act)
    deq = O.dequant_1x128(q.cpu(), s.cpu())
    deq_ref = O.dequant_1x128(q_ref, s_ref)
    assert O.rdiff(deq, deq_ref) < 2e-3
    # identical wherever the rounded activation is identical: the vast majority of bytes
    same = (q.cpu().view(torch.uint8) == q_ref.view(torch.uint8)).float().mean().item()
    assert same > 0.995
    # and the two-kernel GPU path (torch SwiGLU on the GPU, then the plain quantiser) agrees with the fused one
    act_gpu = (torch.nn.functional.silu(h.to(DEV)[:, :256].float()) * h.to(DEV)[:, 256:].float()).bfloat16()
    q2, s2 = per_token_cast_to_fp8(act_gpu)
    assert O.rdiff(O.dequant_1x128(q2.cpu(), s2.cpu()), deq) < 2e-3


def test_gather_and_combine_kernels_are_exact():
    from triton_grouped_gemm_b200.ep.dispatch import combine, dispatch, make_plan

    t, e, k, h = 513, 8, 4, 1024
    idx, w = synthetic_routing(t, e, k, seed=5)
    gen = torch.Generator().manual_seed(6)
    x8 = torch.randn(t, h, generator=gen).to(torch.float8_e4m3fn)
    xs = torch.rand(t, h // 128, generator=gen)
    plan_c = make_plan(idx, e)
    plan_g = make_plan(idx.to(DEV), e)
    # the device plan (counting-sort kernels) groups the pairs by expert like the host's stable sort,
    # in an unspecified order inside each expert: same counts, a permutation, expert ids ascending
    order_g = plan_g.send_order.cpu()
    assert plan_g.size_per_group.cpu().tolist() == plan_c.size_per_group.tolist()
    assert torch.equal(torch.sort(order_g).values, torch.arange(t * k))
    experts_in_order = idx.reshape(-1)[order_g]
    assert bool((experts_in_order[1:] >= experts_in_order[:-1]).all())
    assert torch.equal(plan_g.pos.cpu()[order_g], torch.arange(t * k))
    # gather of byte rows and of fp32 scale rows: identical to torch indexing with the plan's order
    token_of_row = order_g // k
    assert torch.equal(dispatch(plan_g, x8.to(DEV)).cpu().view(torch.uint8), x8.view(torch.uint8)[token_of_row])
    assert torch.equal(dispatch(plan_g, xs.to(DEV)).cpu(), xs[token_of_row])
    # weighted top-k sum: fp32 accumulation, one rounding -> agrees with the host formula to 1 bf16 ulp.
    # y is given in each plan's own row order: row i belongs to pair send_order[i]
    y_pairs = torch.randn(t * k, h, generator=gen).bfloat16()        # indexed by pair (t*k + kk)
    out_g = combine(plan_g, y_pairs[order_g].to(DEV), w.to(DEV)).cpu()
    out_c = combine(plan_c, y_pairs[plan_c.send_order], w)
    assert O.rdiff(out_g.float(), out_c.float()) < 1e-3
    assert (out_g.float() - out_c.float()).abs().max() <= 2 ** -7 * out_c.float().abs().max()


@pytest.mark.parametrize("t,h,inter,e,k", [(96, 256, 128, 4, 2), (300, 512, 256, 8, 3)])
def test_layer_single_rank_vs_oracle(t, h, inter, e, k):
    gen = torch.Generator().manual_seed(t + e)
    x = torch.randn(t, h, generator=gen).bfloat16()
    w13 = (torch.randn(e, 2 * inter, h, generator=gen) * 0.05).bfloat16()
    w2 = (torch.randn(e, h, inter, generator=gen) * 0.05).bfloat16()
    idx, w = synthetic_routing(t, e, k, seed=3)
    ref = O.moe_layer_ref(x, idx, w, w13, w2)
    layer = Fp8MoELayer(w13.to(DEV), w2.to(DEV), e)
    out = layer.forward(x.to(DEV), idx.to(DEV), w.to(DEV)).cpu()
    assert out.shape == ref.shape and out.dtype == torch.bfloat16
    assert O.rdiff(out.float(), ref.float()) < 5e-3


def test_decode_masked_variant():
    e, m_max, h, inter = 4, 128, 256, 128
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(e * m_max, h, generator=gen).bfloat16()
    w13 = (torch.randn(e, 2 * inter, h, generator=gen) * 0.05).bfloat16()
    w2 = (torch.randn(e, h, inter, generator=gen) * 0.05).bfloat16()
    masked = torch.tensor([128, 0, 37, 100])
    layer = Fp8MoELayer(w13.to(DEV), w2.to(DEV), e)
    x8, xs = per_token_cast_to_fp8(x.to(DEV))
    out = layer.decode(x8, xs, masked.to(DEV), m_max).cpu()
    # reference: each valid row through its expert (top-1 routing with weight 1)
    for g, m in enumerate(masked.tolist()):
        rows = slice(g * m_max, g * m_max + m)
        if m:
            idx = torch.full((m, 1), g)
            ref = O.moe_layer_ref(x[rows], idx, torch.ones(m, 1), w13, w2)
            assert O.rdiff(out[rows].float(), ref.float()) < 5e-3
        assert torch.all(out[g * m_max + m:(g + 1) * m_max] == 0)


def test_multi_buffer_row_movers_on_one_gpu():
    """The peer-memory dispatch / combine kernels with three ordinary buffers standing in for the
    ranks' buffers: exact against torch indexing; an out-of-range index is reported, not followed."""
    import ctypes

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator().manual_seed(21)
    t, k, h, world, cap = 257, 4, 512, 3, 600
    x = torch.randn(t, h, generator=gen).to(torch.float8_e4m3fn).view(torch.uint8).to(DEV)
    n = t * k
    src_idx = torch.randint(0, t, (n,), generator=gen).to(DEV)
    dst_rank = torch.randint(0, world, (n,), generator=gen, dtype=torch.int32)
    # distinct rows per rank
    dst_row = torch.empty(n, dtype=torch.int64)
    for r in range(world):
        sel = (dst_rank == r).nonzero().flatten()
        dst_row[sel] = torch.randperm(cap, generator=gen)[: sel.numel()]
    bufs = [torch.zeros(cap, h, dtype=torch.uint8, device=DEV) for _ in range(world)]
    bases = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    rank_d, row_d = dst_rank.to(DEV), dst_row.to(DEV)   # named: the kernels read them after the call returns
    rc = lib.b200moe_scatter_rows_multi(x.data_ptr(), src_idx.data_ptr(), bases, rank_d.data_ptr(),
                                        row_d.data_ptr(), n, h, world, cap, t, 0, stream)
    _lib.check(rc, "scatter")
    torch.cuda.synchronize()
    for r in range(world):
        ref = torch.zeros(cap, h, dtype=torch.uint8)
        sel = dst_rank == r
        ref[dst_row[sel]] = x.cpu()[src_idx.cpu()[sel]]
        assert torch.equal(bufs[r].cpu(), ref)
    # combine: weighted sum of bf16 rows read from the three buffers
    ybufs = [torch.randn(cap, h, generator=gen).bfloat16().to(DEV) for _ in range(world)]
    ybases = (ctypes.c_void_p * world)(*[b.data_ptr() for b in ybufs])
    w = torch.rand(t, k, generator=gen)
    w_d = w.to(DEV)
    out = torch.empty(t, h, dtype=torch.bfloat16, device=DEV)
    rc = lib.b200moe_combine_topk_multi(ybases, rank_d.data_ptr(), row_d.data_ptr(), w_d.data_ptr(), out.data_ptr(),
                                        t, k, h, world, cap, stream)
    _lib.check(rc, "combine")
    rows = torch.stack([ybufs[int(r)].cpu()[int(i)] for r, i in zip(dst_rank.tolist(), dst_row.tolist())]).float()
    ref = (rows.view(t, k, h) * w[:, :, None]).sum(1)
    assert (out.cpu().float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    assert O.rdiff(out.cpu().float(), ref) < 3e-3
    # a row beyond the capacity is skipped and flagged
    bad_row = dst_row.clone()
    bad_row[5] = cap + 7
    bad_row_d = bad_row.to(DEV)
    before = bufs[int(dst_rank[5])].clone()
    rc = lib.b200moe_scatter_rows_multi(x.data_ptr(), src_idx.data_ptr(), bases, rank_d.data_ptr(),
                                        bad_row_d.data_ptr(), n, h, world, cap, t, 0, stream)
    _lib.check(rc, "scatter")
    assert _lib.device_status() == 1 << 5
    assert torch.equal(bufs[int(dst_rank[5])], before)   # same data everywhere else, nothing new written
    # a source row outside src is skipped and flagged too (16 large blocks: the form used beside a GEMM)
    bad_src = src_idx.clone()
    bad_src[9] = t + 3
    bad_src[11] = -1
    for b in bufs:
        b.zero_()
    rc = lib.b200moe_scatter_rows_multi(x.data_ptr(), bad_src.data_ptr(), bases, rank_d.data_ptr(),
                                        row_d.data_ptr(), n, h, world, cap, t, 16, stream)
    _lib.check(rc, "scatter")
    assert _lib.device_status() == 1 << 5
    for r in range(world):
        ref = torch.zeros(cap, h, dtype=torch.uint8)
        sel = (dst_rank == r) & (torch.arange(n) != 9) & (torch.arange(n) != 11)
        ref[dst_row[sel]] = x.cpu()[src_idx.cpu()[sel]]
        assert torch.equal(bufs[r].cpu(), ref)


def test_quantise_on_dispatch_and_return_movers_on_one_gpu():
    """b200moe_dispatch_quant_rows_multi with three ordinary buffers per payload standing in for the
    ranks': the rows, scales and return addresses it stores are bit for bit what the activation
    quantiser followed by one scatter per payload stores.  b200moe_return_rows_multi then sends
    rows back through those addresses.  Both in their GPU-filling and their few-large-blocks form."""
    import ctypes

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator().manual_seed(33)
    t, k, h, world, cap, me = 193, 4, 1024, 3, 400, 1
    x = torch.randn(t, h, generator=gen).bfloat16()
    x[7, 128:256] = 0                      # a block at the 1e-4 clamp
    x[9, :] *= 300.0
    n = t * k
    tok = torch.randint(0, t, (n,), generator=gen)
    dst_rank = torch.randint(0, world, (n,), generator=gen, dtype=torch.int32)
    dst_row = torch.empty(n, dtype=torch.int64)
    for r in range(world):
        sel = (dst_rank == r).nonzero().flatten()
        dst_row[sel] = torch.randperm(cap, generator=gen)[: sel.numel()]
    q_ref, s_ref = O.per_token_cast_to_fp8(x)
    x_d, tok_d, rank_d, row_d = x.to(DEV), tok.to(DEV), dst_rank.to(DEV), dst_row.to(DEV)
    first, count = 5, n - 9                # a sub-range of the send order, as a chunk is
    for blocks in (0, 8):
        b8 = [torch.zeros(cap, h, dtype=torch.uint8, device=DEV) for _ in range(world)]
        bs = [torch.zeros(cap, h // 128, dtype=torch.float32, device=DEV) for _ in range(world)]
        bm = [torch.full((cap, 2), -7, dtype=torch.int64, device=DEV) for _ in range(world)]
        mk = lambda bufs: (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])  # noqa: E731
        rc = lib.b200moe_dispatch_quant_rows_multi(x_d.data_ptr(), tok_d.data_ptr(), mk(b8), mk(bs), mk(bm),
                                                   rank_d.data_ptr(), row_d.data_ptr(), first, count, t, h, 0, world, cap,
                                                   me, blocks, stream)
        _lib.check(rc, "dispatch_quant")
        torch.cuda.synchronize()
        for r in range(world):
            e8 = torch.zeros(cap, h, dtype=torch.uint8)
            es = torch.zeros(cap, h // 128)
            em = torch.full((cap, 2), -7, dtype=torch.int64)
            for i in range(first, first + count):
                if int(dst_rank[i]) == r:
                    e8[dst_row[i]] = q_ref.view(torch.uint8)[tok[i]]
                    es[dst_row[i]] = s_ref[tok[i]]
                    em[dst_row[i]] = torch.tensor([i, me])
            assert torch.equal(b8[r].cpu(), e8)
            assert torch.equal(bs[r].cpu().view(torch.int32), es.view(torch.int32))
            assert torch.equal(bm[r].cpu(), em)
        assert _lib.device_status() == 0
        # the same stores from rows quantised beforehand (b200moe_dispatch_rows_multi)
        q_d, s_d = q_ref.view(torch.uint8).to(DEV), s_ref.to(DEV)
        c8 = [torch.zeros(cap, h, dtype=torch.uint8, device=DEV) for _ in range(world)]
        cs = [torch.zeros(cap, h // 128, dtype=torch.float32, device=DEV) for _ in range(world)]
        cm = [torch.full((cap, 2), -7, dtype=torch.int64, device=DEV) for _ in range(world)]
        rc = lib.b200moe_dispatch_rows_multi(q_d.data_ptr(), s_d.data_ptr(), tok_d.data_ptr(), mk(c8), mk(cs), mk(cm),
                                             rank_d.data_ptr(), row_d.data_ptr(), first, count, t, h, world, cap, me,
                                             blocks, stream)
        _lib.check(rc, "dispatch_rows")
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(c8[r], b8[r]) and torch.equal(cs[r].view(torch.int32), bs[r].view(torch.int32))
            assert torch.equal(cm[r], bm[r])
        assert _lib.device_status() == 0
    # the way back: rows [0, m) of a result buffer go to (meta[r, 1], meta[r, 0])
    m = 300
    y = torch.randn(m, h, generator=gen).bfloat16().to(DEV)
    back_rank = torch.randint(0, world, (m,), generator=gen)
    back_row = torch.empty(m, dtype=torch.int64)
    for r in range(world):
        sel = (back_rank == r).nonzero().flatten()
        back_row[sel] = torch.randperm(cap, generator=gen)[: sel.numel()]
    meta = torch.stack([back_row, back_rank], dim=1).contiguous().to(DEV)
    for blocks in (0, 8):
        rets = [torch.zeros(cap, h, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
        rbases = (ctypes.c_void_p * world)(*[b.data_ptr() for b in rets])
        rc = lib.b200moe_return_rows_multi(y.data_ptr(), meta.data_ptr(), rbases, m, h * 2, world, cap, blocks, stream)
        _lib.check(rc, "return_rows")
        torch.cuda.synchronize()
        for r in range(world):
            ref = torch.zeros(cap, h, dtype=torch.bfloat16)
            sel = back_rank == r
            ref[back_row[sel]] = y.cpu()[sel]
            assert torch.equal(rets[r].cpu(), ref)
    # a return address outside the buffers is skipped and flagged
    meta_bad = meta.clone()
    meta_bad[3, 1] = world
    meta_bad[4, 0] = cap
    rc = lib.b200moe_return_rows_multi(y.data_ptr(), meta_bad.data_ptr(), rbases, m, h * 2, world, cap, 0, stream)
    _lib.check(rc, "return_rows")
    assert _lib.device_status() == 1 << 5


def test_dropped_routing_pair_is_skipped_not_followed():
    """One (token, k) pair with expert id -1 (a dropped token): the routing plan gives it no slot,
    the movers skip it (status bit 5), and the layer's output for that token is the weighted sum of
    its other experts."""
    e, h, inter, k, t = 4, 256, 128, 2, 96
    gen = torch.Generator().manual_seed(8)
    w13 = (torch.randn(e, 2 * inter, h, generator=gen) * 0.05).bfloat16()
    w2 = (torch.randn(e, h, inter, generator=gen) * 0.05).bfloat16()
    x = torch.randn(t, h, generator=gen).bfloat16()
    idx, w = synthetic_routing(t, e, k, seed=3)
    idx[17, 1] = -1
    layer = Fp8MoELayer(w13.to(DEV), w2.to(DEV), e, None)
    out = layer.forward(x.to(DEV), idx.to(DEV), w.to(DEV)).cpu()
    assert _lib.device_status() == 1 << 5
    idx_ok, w_ok = idx.clone(), w.clone()
    idx_ok[17, 1] = idx[17, 0]
    w_ok[17, 1] = 0.0
    ref = layer.forward(x.to(DEV), idx_ok.to(DEV), w_ok.to(DEV)).cpu()
    assert _lib.device_status() == 0
    assert torch.equal(out, ref)


@pytest.mark.parametrize("t,h,k,dtype", [(257, 512, 4, torch.bfloat16), (96, 4096, 8, torch.bfloat16),
                                          (65, 8192, 2, torch.float16), (33, 128, 1, torch.bfloat16)])
def test_quantise_and_permute_in_one_pass_is_bit_exact(t, h, k, dtype):
    """b200moe_quant_scatter_rows against the quantiser followed by the gather: same bytes, same
    scales at every row a pair owns; a dropped pair (pos = -1) is skipped and flagged."""
    from triton_grouped_gemm_b200.ep.dispatch import dispatch, make_plan, quant_permute_rows

    e = 8
    idx, _ = synthetic_routing(t, e, k, seed=31)
    if t > 40:
        idx[7, 0] = -1
    gen = torch.Generator().manual_seed(32)
    x = (torch.randn(t, h, generator=gen) * torch.rand(t, 1, generator=gen) * 3).to(dtype).to(DEV)
    x[3] = 0                                  # an all-zero row: scale floor
    plan = make_plan(idx.to(DEV), e)
    _lib.device_status()
    r8, rs = quant_permute_rows(x, plan.pos, k)
    status = _lib.device_status()
    assert status == ((1 << 5) if t > 40 else 0)
    x8, xs = per_token_cast_to_fp8(x)
    g8, gs = dispatch(plan, x8), dispatch(plan, xs)
    status = _lib.device_status()             # the gather skips the dropped pair's slot too
    n_ok = int(((idx >= 0) & (idx < e)).sum())
    assert torch.equal(r8[:n_ok].view(torch.uint8), g8[:n_ok].view(torch.uint8))
    assert torch.equal(rs[:n_ok], gs[:n_ok])
    # and against the oracle's quantiser at the rows of a few pairs
    ref8, refs = O.per_token_cast_to_fp8(x.cpu())
    pos = plan.pos.cpu()
    for pair in (0, t * k // 2, t * k - 1):
        if pos[pair] >= 0:
            assert torch.equal(r8[pos[pair]].cpu().view(torch.uint8), ref8[pair // k].view(torch.uint8))
            assert torch.equal(rs[pos[pair]].cpu(), refs[pair // k])


def test_peer_plan_kernels_match_the_host_formulas():
    """b200moe_route_plan_mapped + b200moe_peer_plan for three pretended ranks on one GPU: counts in
    key order, the [local expert][source rank] row of every pair and the per-expert row counts equal
    what plain indexing gives."""
    import numpy as np

    from triton_grouped_gemm_b200.ep.p2p import _key_tables, chunk_bounds

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    world, e_loc, k = 3, 4, 2
    E = world * e_loc
    bounds = chunk_bounds(e_loc, 3)                      # uneven chunks of the local experts
    key_h, inv_h, key_d, inv_d = _key_tables(world, e_loc, tuple(bounds), torch.device(DEV))
    gen = torch.Generator().manual_seed(12)
    routing = [torch.randint(0, E, (37 + 5 * r, k), generator=gen) for r in range(world)]
    routing[2][4, 1] = -1                                # a dropped pair on rank 2
    counts, orders, flats = [], [], []
    for r in range(world):
        flat = routing[r].reshape(-1).to(DEV)
        n = flat.numel()
        c = torch.empty(E, dtype=torch.int32, device=DEV)
        cur = torch.empty(E, dtype=torch.int32, device=DEV)
        order = torch.empty(n, dtype=torch.int64, device=DEV)
        pos = torch.empty(n, dtype=torch.int64, device=DEV)
        _lib.check(lib.b200moe_route_plan_mapped(flat.data_ptr(), n, E, key_d.data_ptr(), c.data_ptr(), cur.data_ptr(),
                                                 order.data_ptr(), pos.data_ptr(), stream), "route_plan_mapped")
        counts.append(c)
        orders.append(order)
        flats.append(flat)
        ok = (routing[r].reshape(-1) >= 0)
        ref_counts = np.bincount(key_h[routing[r].reshape(-1)[ok].numpy()], minlength=E)
        assert c.cpu().tolist() == ref_counts.tolist()
    assert _lib.device_status() == 1 << 5                # the dropped pair was flagged
    counts_all = torch.stack(counts).contiguous()        # [s, key]
    ca = counts_all.cpu().numpy()[:, key_h].reshape(world, world, e_loc)   # [s, d, l]
    for me in range(world):
        n = flats[me].numel()
        scratch = torch.empty(2 * E + e_loc, dtype=torch.int64, device=DEV)
        tok = torch.empty(n, dtype=torch.int64, device=DEV)
        dr = torch.empty(n, dtype=torch.int32, device=DEV)
        drow = torch.empty(n, dtype=torch.int64, device=DEV)
        _lib.check(lib.b200moe_peer_plan(counts_all.data_ptr(), inv_d.data_ptr(), key_d.data_ptr(), world, me, E,
                                         orders[me].data_ptr(), flats[me].data_ptr(), n, k, scratch.data_ptr(),
                                         scratch[E:].data_ptr(), scratch[2 * E:].data_ptr(), tok.data_ptr(),
                                         dr.data_ptr(), drow.data_ptr(), stream), "peer_plan")
        torch.cuda.synchronize()
        assert scratch[2 * E:].cpu().tolist() == ca[:, me, :].sum(axis=0).tolist()          # rows per local expert
        order = orders[me].cpu().numpy()
        flat = flats[me].cpu().numpy()
        my_counts = counts_all[me].cpu().numpy()
        send_start = my_counts.cumsum() - my_counts
        seen = {}
        for i in range(n):
            p = order[i]
            if p < 0:
                assert tok[i].item() == -1 and dr[i].item() == -1
                continue
            e = flat[p]
            d, l = divmod(e, e_loc)
            key = key_h[e]
            before = ca[:, d, :l].sum() + ca[:me, d, l].sum()                               # [l][s] layout at rank d
            assert tok[i].item() == p // k and dr[i].item() == d
            assert drow[i].item() == before + (i - send_start[key])
            assert (d, drow[i].item()) not in seen
            seen[(d, drow[i].item())] = True
