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
                                        row_d.data_ptr(), n, h, world, cap, stream)
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
                                        bad_row_d.data_ptr(), n, h, world, cap, stream)
    _lib.check(rc, "scatter")
    assert _lib.device_status() == 1 << 5
    assert torch.equal(bufs[int(dst_rank[5])], before)   # same data everywhere else, nothing new written
