"""Expert-parallel dispatch / combine on CPU: single process, and two gloo ranks exchanging
rows, checked against a direct per-token computation."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from triton_grouped_gemm_b200.ep.dispatch import combine, dispatch, make_plan
from triton_grouped_gemm_b200.ep.moe_layer import synthetic_routing


def _expert_fn(rows: torch.Tensor, sizes: torch.Tensor, first_expert: int) -> torch.Tensor:
    """Toy per-expert computation: row * (global expert id + 1)."""
    out = torch.empty_like(rows)
    start = 0
    for e, n in enumerate(sizes.tolist()):
        out[start:start + n] = rows[start:start + n] * float(first_expert + e + 1)
        start += n
    return out


def _reference(x, idx, w):
    return (x[:, None, :] * (idx[:, :, None].float() + 1.0) * w[:, :, None]).sum(1)


def test_single_rank_roundtrip():
    t, e, k, h = 37, 8, 3, 16
    idx, w = synthetic_routing(t, e, k, seed=1)
    x = torch.randn(t, h)
    plan = make_plan(idx, e)
    rows = dispatch(plan, x)
    assert rows.shape == (t * k, h) and int(plan.size_per_group.sum()) == t * k
    assert plan.size_per_group.tolist() == torch.bincount(idx.reshape(-1), minlength=e).tolist()
    y = combine(plan, _expert_fn(rows, plan.size_per_group, 0), w)
    assert torch.allclose(y, _reference(x, idx, w), atol=1e-5)
    # byte payloads (fp8) travel unchanged
    b = torch.randn(t, h).to(torch.float8_e4m3fn)
    rb = dispatch(plan, b)
    assert rb.dtype == torch.float8_e4m3fn
    token_of_row = (plan.send_order // k)[plan.recv_to_expert_major]
    assert torch.equal(rb.view(torch.uint8), b.view(torch.uint8)[token_of_row])


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        t, e, k, h = 29 + 5 * rank, 8, 2, 8
        idx, w = synthetic_routing(t, e, k, seed=10 + rank)
        gen = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(t, h, generator=gen)
        plan = make_plan(idx, e, dist.group.WORLD)
        rows = dispatch(plan, x, dist.group.WORLD)
        e_loc = e // world
        # every received row must belong to one of this rank's experts, in expert-major order
        assert int(plan.size_per_group.sum()) == rows.shape[0]
        y = combine(plan, _expert_fn(rows, plan.size_per_group, rank * e_loc), w, dist.group.WORLD)
        ok = torch.allclose(y, _reference(x, idx, w), atol=1e-5)
        # total rows over all ranks == total routed pairs
        tot = torch.tensor([rows.shape[0], t * k])
        dist.all_reduce(tot)
        results[rank] = bool(ok) and int(tot[0]) == int(tot[1])
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert results.get(0) is True and results.get(1) is True
