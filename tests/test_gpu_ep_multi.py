"""Expert-parallel FP8 layer on two GPUs (skipped on a single-GPU box): both transports - NCCL
all-to-all and the peer-memory row movers - must reproduce the single-rank layer exactly, over
several steps that reuse the exchange buffers; each transport in its one-shot form (chunks = 1)
and pipelined over groups of local experts (4 even groups; for peer memory also 3 uneven ones
and 8, with the dispatch kernel quantising the bf16 rows itself; results going home by copy
engine or by the return-address mover kernel).  The peer-memory layers are
closed collectively before the process group goes away."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, transport, chunks, qod, return_path, dispatch_path, results):
    import torch.distributed as dist

    from triton_grouped_gemm_b200 import _lib
    from triton_grouped_gemm_b200.ep.moe_layer import Fp8MoELayer, synthetic_routing

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        e, h, inter, k, t = 16, 512, 256, 4, 1024
        g = torch.Generator().manual_seed(0)
        w13 = (torch.randn(e, 2 * inter, h, generator=g) * 0.05).bfloat16()
        w2 = (torch.randn(e, h, inter, generator=g) * 0.05).bfloat16()
        e_loc = e // world
        layer = Fp8MoELayer(w13[rank * e_loc:(rank + 1) * e_loc].to(dev), w2[rank * e_loc:(rank + 1) * e_loc].to(dev), e,
                            dist.group.WORLD, transport=transport, chunks=chunks, tokens_per_rank=t, top_k=k,
                            capacity_factor=2.0, quantise_on_dispatch=qod, return_path=return_path,
                            dispatch_path=dispatch_path)
        full = Fp8MoELayer(w13.to(dev), w2.to(dev), e, None)
        worst = 0.0
        for step in range(3):
            gx = torch.Generator().manual_seed(100 + rank + 10 * step)
            x = torch.randn(t, h, generator=gx).bfloat16().to(dev)
            idx, w = synthetic_routing(t, e, k, seed=200 + rank + 10 * step)
            out = layer.forward(x, idx.to(dev), w.to(dev))
            ref = full.forward(x, idx.to(dev), w.to(dev))
            worst = max(worst, ((out.float() - ref.float()).abs().sum() / ref.float().abs().sum()).item())
        status = _lib.device_status()
        layer.close()          # collective: waits for the device, barriers, then unmaps and frees
        layer.close()          # a second call is a no-op
        results[rank] = (worst, status)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("transport,chunks,qod,return_path,dispatch_path", [
    ("p2p", 1, False, "copy", "copy"), ("p2p", 4, False, "copy", "copy"), ("p2p", 3, False, "copy", "copy"),
    ("p2p", 4, False, "copy", "kernel"), ("p2p", 3, True, "copy", "kernel"), ("p2p", 8, True, "kernel", "kernel"),
    ("p2p", 4, False, "kernel", "kernel"), ("nccl", 1, False, "copy", "copy"), ("nccl", 4, False, "copy", "copy")])
def test_two_gpu_layer_matches_single_rank(transport, chunks, qod, return_path, dispatch_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, transport, chunks, qod, return_path, dispatch_path, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
            assert p.exitcode == 0
        for r in range(2):
            worst, status = results[r]
            assert worst == 0.0 and status == 0
