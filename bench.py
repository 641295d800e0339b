#!/usr/bin/env python
"""Benchmark of the grouped-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

One "step" = one pass of the hot path over one batch: a single M-grouped GEMM launch over all
experts a rank owns.  Default workload (``bf16_m_grouped_gate_up``): G=128 experts, 655 360
routed rows (multinomial over softmax(N(0,0.5)) logits, each expert padded to 128 rows),
K=2048, N=1536, trans_b=True, A and B ~ N(0,1)*0.02 in bf16, synthetic and seeded.  With N>1
ranks (torchrun, one per GPU) the experts are partitioned G/N per rank and every rank keeps
655 360 routed rows (weak scaling, no data-path collective; the only collectives are the
barrier and the max-over-ranks of the timing).

Prints ONE JSON line (rank 0).  ``value`` = device-timed TFLOP/s with inputs resident in HBM;
``e2e`` = the same metric through the public Python operator with HOST (pinned) inputs and a
host result, copies inside the timed region.  ``--impl reference`` times the reference's CPU
path (torch per-group loop, restated in oracle/) on this host's cores on a bounded sample.

Beside the headline the default line carries (``--no-extras`` drops them):
  roofline.sustained  the same step back to back for >= 2 s (power-capped clocks, sampled)
  also                the FP8 block-scaled gate+up GEMM (K=4096, N=3072) on the same routing, with a
                      parity figure against the CPU oracle taken inside the run
  gpu_reference       N=1 only: the reference's own Triton kernel, autotuned, timed in a child
                      process on the same sizes when an installed copy sits in baseline/_ref
  ep                  N>1 only: the expert-parallel FP8 MoE layer (81 920 tokens per rank, top-8) on
                      the same process group, both transports, with its result compared to the
                      single-rank layer, and the masked decode step
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (kind, K, N, trans_b)
    "bf16_m_grouped_gate_up": ("m_grouped", 2048, 1536, True),
    "bf16_m_grouped_gate_up_nn": ("m_grouped", 2048, 1536, False),
    # the reference's own benchmark case (gemm/BF16/m_grouped_gemm_TMA.py:474-493 of the reference):
    # 128 uniform groups of 5120 rows, N(0,1) data - like for like with its README / its B200 run
    "bf16_m_grouped_uniform": ("m_grouped", 2048, 1536, True),
    "bf16_m_grouped_uniform_down": ("m_grouped", 768, 2048, True),
    "bf16_m_grouped_down": ("m_grouped", 768, 2048, True),
    "bf16_k_grouped_wgrad": ("k_grouped", 2048, 768, False),
    "fp8_block_m_grouped_gate_up": ("fp8_block", 4096, 3072, True),
    "fp8_block_m_grouped_down": ("fp8_block", 1536, 4096, True),
    # FP8 with per-row x per-channel scales (e4m3 x e4m3), M-grouped and K-grouped (tokens padded to 128)
    "fp8_rowcol_m_grouped": ("fp8_rowcol", 4096, 3072, True),
    "fp8_rowcol_k_grouped": ("fp8_rowcol_k", 2048, 768, False),
    # FP8 weight gradient: both operands from the transposing 128x128 quantiser, 2048 x 768 per expert
    "fp8_block_k_grouped_wgrad": ("fp8_block_k", 2048, 768, False),
    # masked layout: 128 slots of 4096 rows, ~1/4 of them valid (the reference's masked benchmark)
    "bf16_masked_m_grouped": ("masked", 2048, 1536, True),
    "quant_act_1x128": ("quant_act", 4096, 0, True),
    # the one-GPU MoE layer's first step: 1x128 quantiser + token permute in one pass (rows / 8 tokens, top-8)
    "quant_permute_1x128": ("quant_permute", 4096, 0, True),
    # transposing 128x128 quantiser with per-expert expansion: input [rows, 4096] bf16
    "quant_trans_expand_128x": ("quant_trans", 4096, 0, True),
    # expert-parallel FP8 MoE layer: K = hidden 4096, N = intermediate 1536, 128 experts, top-8,
    # --rows = routed rows per GPU (tokens per GPU = rows / 8); NCCL all-to-all dispatch + combine
    "moe_ep_fp8": ("moe_ep", 4096, 1536, True),
    # decode: masked layout [experts per GPU, 256 slots], valid counts uniform in [0, 256]
    "moe_decode_fp8": ("moe_decode", 4096, 1536, True),
}
TOP_K = 8
DECODE_M_MAX = 256
TOTAL_ROWS = 655360
NUM_EXPERTS = 128
ROUTING_SEED = 2026
ROWS_USED = [TOTAL_ROWS]
UNIFORM_WORKLOADS = ("bf16_m_grouped_uniform", "bf16_m_grouped_uniform_down")
UNIFORM = [False]
DATA_SCALE = [0.02]  # std of the 16-bit GEMM operands; the uniform workloads use the reference's N(0,1)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"bf16": float(d["bf16_tflops"]), "bf16_sustained": float(d.get("bf16_tflops_sustained", 0) or 0),
                    "hbm": float(d["hbm_gbs"]), "source": "measured"}
        except Exception:
            pass
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    QUERY = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, t_begin=None, t_end=None):
        """Summarise the samples; with wall-clock bounds only those taken inside the timed region
        (if there are any) are used for the median clock and the throttle reasons."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        import datetime

        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[2]), float(parts[3]), float(parts[4]),
                             [n for n, v in zip(names, parts[6:10]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if t_begin is not None and t_begin - 0.02 <= r[0] <= t_end + 0.02]
        use = inside or rows
        reasons = sorted({n for r in use for n in r[4]})
        return {"sm_mhz": statistics.median([r[1] for r in use]) if use else None,
                "sm_max_mhz": max([r[2] for r in use]) if use else None,
                "power_w": statistics.median([r[3] for r in use]) if use else None,
                "reasons": reasons, "samples": len(use), "samples_in_timed_region": len(inside)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def rank_sizes(world: int, rank: int, total_rows: int = TOTAL_ROWS, experts: int = NUM_EXPERTS) -> torch.Tensor:
    """Row counts of the experts this rank owns.  Every rank keeps `total_rows` routed rows over
    its experts/world experts (routing seed varies with the rank)."""
    g_local = max(experts // world, 1)
    if UNIFORM[0]:
        return torch.full((g_local,), total_rows // g_local, dtype=torch.int64)
    gen = torch.Generator().manual_seed(ROUTING_SEED + rank)
    logits = 0.5 * torch.randn(g_local, generator=gen)
    draws = torch.multinomial(torch.softmax(logits, dim=0), total_rows, replacement=True, generator=gen)
    counts = torch.bincount(draws, minlength=g_local)
    return ((counts + 127) // 128 * 128).to(torch.int64)


def moe_sizes(kind, world, rank, rows):
    """moe_ep: nominal rows per local expert (only the count of local experts matters; the real
    sizes come from the routing at run time).  moe_decode: valid rows per local expert slot."""
    e_loc = NUM_EXPERTS // world
    if kind == "moe_ep":
        return torch.full((e_loc,), rows // e_loc, dtype=torch.int64)
    gen = torch.Generator().manual_seed(ROUTING_SEED + rank)
    return torch.randint(0, DECODE_M_MAX + 1, (e_loc,), generator=gen, dtype=torch.int64)


def make_inputs(kind, k, n, trans_b, sizes, device, seed):
    gen = torch.Generator(device=device).manual_seed(seed)
    m = int(sizes.sum())
    g = sizes.numel()

    def randn(shape, scale, chunk_rows=65536):
        out = torch.empty(shape, device=device, dtype=torch.bfloat16)
        flat = out.view(shape[0], -1)
        for r in range(0, shape[0], chunk_rows):
            rows = min(chunk_rows, shape[0] - r)
            flat[r:r + rows] = (torch.randn(rows, flat.shape[1], device=device, generator=gen) * scale).bfloat16()
        return out

    if kind == "m_grouped":
        a = randn((m, k), DATA_SCALE[0])
        b = randn((g, n, k) if trans_b else (g, k, n), DATA_SCALE[0], chunk_rows=8)
        return {"a": a, "b": b}
    if kind == "k_grouped":
        return {"a": randn((m, k), 0.02), "b": randn((m, n), 0.02)}
    if kind == "fp8_block":
        return {"x": randn((m, k), 1.0), "w": randn((g, n, k), 0.02, chunk_rows=4)}
    if kind in ("quant_act", "quant_trans"):
        return {"x": randn((m, k), 1.0)}
    if kind == "quant_permute":
        return {"x": randn((m // TOP_K, k), 1.0)}
    if kind == "fp8_rowcol":
        a8 = (randn((m, k), 100.0).float().clamp(-400, 400)).to(torch.float8_e4m3fn)
        b8 = (randn((g, n, k), 100.0, chunk_rows=4).float().clamp(-400, 400)).to(torch.float8_e4m3fn)
        return {"a8": a8, "a_s": torch.rand(m, device=device, generator=gen) * 0.01 + 1e-3, "b8": b8,
                "b_s": torch.rand(g * n, device=device, generator=gen) * 0.01 + 1e-3}
    if kind == "fp8_rowcol_k":
        # x [M=k, K_total], y [N=n, K_total]; scales group-major [G, M] / [G, N]
        x8 = (randn((k, m), 50.0, chunk_rows=256).float().clamp(-400, 400)).to(torch.float8_e4m3fn)
        y8 = (randn((n, m), 50.0, chunk_rows=256).float().clamp(-400, 400)).to(torch.float8_e4m3fn)
        return {"x8": x8, "y8": y8, "xs": (torch.rand(g, k, device=device, generator=gen) * 0.01 + 1e-3).t(),
                "ys": (torch.rand(g, n, device=device, generator=gen) * 0.01 + 1e-3).t()}
    if kind == "fp8_block_k":
        return {"a": randn((m, k), 1.0), "dy": randn((m, n), 0.1)}
    if kind == "masked":
        e = 4096
        return {"a": randn((g * e, k), 0.02), "b": randn((g, n, k), 0.02, chunk_rows=8)}
    if kind in ("moe_ep", "moe_decode"):
        # sizes = this rank's local-expert placeholder vector; k = hidden, n = intermediate
        return {"w13": randn((g, 2 * n, k), 0.02, chunk_rows=2), "w2": randn((g, k, n), 0.02, chunk_rows=2)}
    raise ValueError(kind)


def algorithmic_work(kind, k, n, sizes):
    rows = int(sizes.sum())
    if kind in ("m_grouped", "fp8_block", "fp8_rowcol", "fp8_rowcol_k", "masked", "fp8_block_k"):
        return 2.0 * rows * n * k, "flop"
    if kind == "k_grouped":
        return 2.0 * rows * n * k, "flop"  # M_DIM=k, N_DIM=n, K_total=rows
    if kind == "quant_act":
        return rows * k * 3.0 + rows * (k // 128) * 4.0, "byte"
    if kind == "quant_permute":
        pairs = rows // TOP_K * TOP_K   # every token's 16-bit row read once, its fp8 row and scales written top_k times
        return pairs // TOP_K * k * 2.0 + pairs * k * 1.0 + pairs * (k // 128) * 4.0, "byte"
    if kind == "quant_trans":
        m_expand = rows + 128 * sizes.numel() - rows % 128
        return rows * k * 2.0 + k * m_expand * 1.0 + (k // 128) * (m_expand // 128) * 4.0, "byte"
    if kind in ("moe_ep", "moe_decode"):
        # gate+up [2n x k] and down [k x n] GEMMs for every routed / valid row
        return 2.0 * rows * (2 * n * k + k * n), "flop"
    raise ValueError(kind)


EP_CHUNKS = 8  # set from --ep-chunks
EP_TRANSPORT = "p2p"  # set from --ep-transport
EP_COMM_SMS = None  # set from --ep-comm-sms (None: the layer's default)


def build_step(kind, k, n, trans_b, sizes_dev, inp):
    """Returns (fn, launches_per_step).  fn() runs one step on the current stream."""
    import triton_grouped_gemm_b200 as pkg  # noqa: F401

    if kind == "m_grouped":
        from triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_TMA import _m_grouped_gemm_launch

        a, b = inp["a"], inp["b"]
        c = torch.empty(a.shape[0], n, device=a.device, dtype=a.dtype)
        inp["c"] = c
        return (lambda: _m_grouped_gemm_launch(a, b, c, sizes_dev, trans_b)), 1
    if kind == "k_grouped":
        from triton_grouped_gemm_b200.gemm.BF16.k_grouped_gemm_TMA import k_grouped_gemm

        a, b = inp["a"], inp["b"]
        return (lambda: inp.__setitem__("c", k_grouped_gemm(a, b, sizes_dev))), 1
    if kind == "fp8_block":
        from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_block_scaled import m_grouped_fp8_block_scaled
        from triton_grouped_gemm_b200.quant.per_block_cast import per_block_cast_to_fp8, per_token_cast_to_fp8

        a8, a_s = per_token_cast_to_fp8(inp["x"])
        b8, b_s = per_block_cast_to_fp8(inp["w"])
        del inp["x"], inp["w"]
        out = torch.empty(a8.shape[0], n, device=a8.device, dtype=torch.bfloat16)
        inp.update(a8=a8, a_s=a_s, b8=b8, b_s=b_s, c=out)
        return (lambda: m_grouped_fp8_block_scaled((a8, a_s), (b8, b_s), sizes_dev, out=out)), 1
    if kind == "quant_act":
        from triton_grouped_gemm_b200.quant.per_block_cast import per_token_cast_to_fp8

        x = inp["x"]
        return (lambda: inp.__setitem__("c", per_token_cast_to_fp8(x))), 1
    if kind == "quant_permute":
        from triton_grouped_gemm_b200.ep.dispatch import make_plan, quant_permute_rows
        from triton_grouped_gemm_b200.ep.moe_layer import synthetic_routing

        x = inp["x"]
        idx, _ = synthetic_routing(x.shape[0], NUM_EXPERTS, TOP_K, seed=ROUTING_SEED, device=x.device)
        pos = make_plan(idx, NUM_EXPERTS).pos
        inp["pos"] = pos
        return (lambda: inp.__setitem__("c", quant_permute_rows(x, pos, TOP_K))), 1
    if kind == "fp8_rowcol":
        from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_channel_expert import gmm_fp8_act_per_channel_w_per_expert as op

        a8, a_s, b8, b_s = inp["a8"], inp["a_s"], inp["b8"], inp["b_s"]
        s32 = sizes_dev.to(torch.int32)
        return (lambda: inp.__setitem__("c", op(a8, a_s, b8, b_s, s32, torch.bfloat16))), 1
    if kind == "fp8_rowcol_k":
        from triton_grouped_gemm_b200.gemm.FP8.k_grouped_gemm_channel_expert import matmul

        x8, y8, xs, ys = inp["x8"], inp["y8"], inp["xs"], inp["ys"]
        s32 = sizes_dev.to(torch.int32)
        return (lambda: inp.__setitem__("c", matmul(x8, xs, y8, ys, s32, k, n, x8.shape[1], s32.numel()))), 1
    if kind == "fp8_block_k":
        from triton_grouped_gemm_b200.gemm.FP8.k_grouped_gemm_block_scaled import k_grouped_fp8_block_scaled
        from triton_grouped_gemm_b200.quant.trans_per_block_quant_expand_128x import trans_per_block_quant_expand_128x

        if "aq" not in inp:  # quantise once, outside the timed region (the quantiser has its own workload)
            aq, a_s, padded = trans_per_block_quant_expand_128x(inp.pop("a"), sizes_dev)
            gq, g_s, _ = trans_per_block_quant_expand_128x(inp.pop("dy"), sizes_dev)
            inp.update(aq=aq, a_s=a_s, gq=gq, g_s=g_s, padded=padded)
        aq, a_s, gq, g_s, padded = inp["aq"], inp["a_s"], inp["gq"], inp["g_s"], inp["padded"]
        return (lambda: inp.__setitem__("c", k_grouped_fp8_block_scaled((aq, a_s), (gq, g_s), padded))), 1
    if kind == "masked":
        from triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_masked_TMA import m_grouped_gemm_masked

        a, b = inp["a"], inp["b"]
        out = torch.empty(a.shape[0], n, device=a.device, dtype=a.dtype)
        inp["c"] = out
        return (lambda: m_grouped_gemm_masked(a, b, out, sizes_dev, 4096, True)), 1
    if kind == "quant_trans":
        from triton_grouped_gemm_b200.quant.trans_per_block_quant_expand_128x import trans_per_block_quant_expand_128x

        x = inp["x"]
        return (lambda: inp.__setitem__("c", trans_per_block_quant_expand_128x(x, sizes_dev))), 1
    if kind in ("moe_ep", "moe_decode"):
        import torch.distributed as dist

        from triton_grouped_gemm_b200.ep.moe_layer import Fp8MoELayer, synthetic_routing
        from triton_grouped_gemm_b200.quant.per_block_cast import per_token_cast_to_fp8

        group = dist.group.WORLD if dist.is_initialized() else None
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        dev = inp["w13"].device
        layer = Fp8MoELayer(inp.pop("w13"), inp.pop("w2"), NUM_EXPERTS if kind == "moe_ep" else sizes_dev.numel(), group,
                            chunks=EP_CHUNKS, comm_sms=EP_COMM_SMS, transport=EP_TRANSPORT if kind == "moe_ep" else "nccl",
                            tokens_per_rank=ROWS_USED[0] // TOP_K, top_k=TOP_K)
        inp["layer"] = layer
        gen = torch.Generator(device=dev).manual_seed(500 + rank)
        if kind == "moe_ep":
            tokens = ROWS_USED[0] // TOP_K
            x = torch.randn(tokens, k, device=dev, generator=gen, dtype=torch.bfloat16)
            idx, w = synthetic_routing(tokens, NUM_EXPERTS, TOP_K, seed=ROUTING_SEED + rank, device=dev)
            inp.update(x=x, idx=idx, w=w)
            # kernels of this library per step on one rank: routing plan (3), quantise-and-permute, two GEMMs,
            # SwiGLU quantiser, weighted combine (more with several ranks: per-chunk movers)
            return (lambda: inp.__setitem__("c", layer.forward(x, idx, w))), 8
        e_loc = sizes_dev.numel()
        x = torch.randn(e_loc * DECODE_M_MAX, k, device=dev, generator=gen, dtype=torch.bfloat16)
        x8, xs = per_token_cast_to_fp8(x)
        out = torch.zeros(e_loc * DECODE_M_MAX, k, device=dev, dtype=torch.bfloat16)
        inp.update(x8=x8, xs=xs, out=out)
        return (lambda: layer.decode(x8, xs, sizes_dev, DECODE_M_MAX, out=out)), 3
    raise ValueError(kind)


def cpu_reference_step(kind, k, n, trans_b, sizes, budget_work, seed=7):
    """The reference's CPU path on a bounded sample: the first groups of the workload whose
    algorithmic work adds up to ~budget_work.  Returns (fn, work_of_sample, description)."""
    import oracle as O

    picked, work = [], 0.0
    for s in sizes.tolist():
        if picked and work >= budget_work:
            break
        picked.append(int(s))
        work += algorithmic_work(kind, k, n, torch.tensor([s]))[0]
    ps = torch.tensor(picked, dtype=torch.int64)
    gen = torch.Generator().manual_seed(seed)
    m = int(ps.sum())
    g = len(picked)
    if kind == "m_grouped":
        a = (torch.randn(m, k, generator=gen) * 0.02).bfloat16()
        b = (torch.randn(g, n, k, generator=gen) * 0.02).bfloat16()
        if not trans_b:
            b = b.transpose(1, 2).contiguous()
        fn = lambda: O.m_grouped_ref(a, b, ps, trans_b)  # noqa: E731
    elif kind == "k_grouped":
        a = (torch.randn(m, k, generator=gen) * 0.02).bfloat16()
        b = (torch.randn(m, n, generator=gen) * 0.02).bfloat16()
        fn = lambda: O.k_grouped_ref(a, b, ps)  # noqa: E731
    elif kind == "fp8_block":
        x = torch.randn(m, k, generator=gen).bfloat16()
        w = (torch.randn(g, n, k, generator=gen) * 0.02).bfloat16()
        a8, a_s = O.per_token_cast_to_fp8(x)
        qs = [O.per_block_cast_to_fp8(w[i]) for i in range(g)]
        b8 = torch.stack([q for q, _ in qs])
        b_s = torch.stack([s for _, s in qs])
        fn = lambda: O.fp8_block_m_grouped_ref(a8, a_s, b8, b_s, ps)  # noqa: E731
    elif kind == "fp8_rowcol":
        a8 = (torch.randn(m, k, generator=gen) * 100).clamp(-400, 400).to(torch.float8_e4m3fn)
        b8 = (torch.randn(g, n, k, generator=gen) * 100).clamp(-400, 400).to(torch.float8_e4m3fn)
        a_s, b_s = torch.rand(m, generator=gen) * 0.01 + 1e-3, torch.rand(g * n, generator=gen) * 0.01 + 1e-3
        fn = lambda: O.fp8_rowcol_m_grouped_ref(a8, a_s, b8, b_s, ps, torch.bfloat16)  # noqa: E731
    elif kind == "fp8_rowcol_k":
        x8 = (torch.randn(k, m, generator=gen) * 50).clamp(-400, 400).to(torch.float8_e4m3fn)
        y8 = (torch.randn(n, m, generator=gen) * 50).clamp(-400, 400).to(torch.float8_e4m3fn)
        xs, ys = (torch.rand(g, k, generator=gen) * 0.01 + 1e-3).t(), (torch.rand(g, n, generator=gen) * 0.01 + 1e-3).t()
        fn = lambda: O.fp8_rowcol_k_grouped_ref(x8, xs, y8, ys, ps, k, n, g)  # noqa: E731
    elif kind == "fp8_block_k":
        a = torch.randn(m, k, generator=gen).bfloat16()
        dy = (torch.randn(m, n, generator=gen) * 0.1).bfloat16()
        aq, a_s, pad = O.trans_quant_expand_ref(a, ps)
        gq, g_s, _ = O.trans_quant_expand_ref(dy, ps)
        fn = lambda: O.fp8_block_k_grouped_ref(aq, a_s, gq, g_s, pad)  # noqa: E731
    elif kind == "masked":
        e = 4096
        a = (torch.randn(g * e, k, generator=gen) * 0.02).bfloat16()
        b = (torch.randn(g, n, k, generator=gen) * 0.02).bfloat16()
        out0 = torch.zeros(g * e, n, dtype=torch.bfloat16)
        fn = lambda: O.m_grouped_masked_ref(a, b, out0, ps, e)  # noqa: E731
    elif kind == "quant_act":
        x = torch.randn(m, k, generator=gen).bfloat16()
        fn = lambda: O.per_token_cast_to_fp8(x)  # noqa: E731
    elif kind == "quant_permute":
        x = torch.randn(m // TOP_K, k, generator=gen).bfloat16()
        order = torch.randperm(m // TOP_K * TOP_K, generator=gen) // TOP_K   # token of every expert-major row

        def fn():
            q, sc = O.per_token_cast_to_fp8(x)
            return q.view(torch.uint8)[order], sc[order]
    elif kind == "quant_trans":
        x = torch.randn(m, k, generator=gen).bfloat16()
        fn = lambda: O.trans_quant_expand_ref(x, ps)  # noqa: E731
    elif kind in ("moe_ep", "moe_decode"):
        # the whole layer on a small token sample routed over 8 experts (fp32 loops on the host)
        tokens, e_s = 256, 8
        x = torch.randn(tokens, k, generator=gen).bfloat16()
        w13 = (torch.randn(e_s, 2 * n, k, generator=gen) * 0.02).bfloat16()
        w2 = (torch.randn(e_s, k, n, generator=gen) * 0.02).bfloat16()
        logits = 0.5 * torch.randn(tokens, e_s, generator=gen)
        wts, idx = torch.topk(torch.softmax(logits, -1), 2, dim=-1)
        fn = lambda: O.moe_layer_ref(x, idx, wts, w13, w2)  # noqa: E731
        work = 2.0 * tokens * 2 * (2 * n * k + k * n)
        desc = (f"{tokens} tokens, top-2 over {e_s} experts of the layer (weights quantised inside the timed call), "
                f"torch {torch.__version__} on host cores")
        return fn, work, desc
    else:
        raise ValueError(kind)
    desc = f"first {g} of {sizes.numel()} groups ({m} rows) of the workload, torch {torch.__version__} on host cores"
    return fn, work, desc


def unit_of(kind):
    return ("TFLOP/s", 1e12) if kind not in ("quant_act", "quant_trans", "quant_permute") else ("GB/s", 1e9)


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU legs are the only host work while
    they run, so give them every core the process may run on."""
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))


def timed_steps(step, steps, warmup):
    """W untimed + K timed steps on the current stream, one CUDA-event pair per step (ms each)."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s_ev, e_ev in evs:
        s_ev.record()
        step()
        e_ev.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


def sustained_leg(step, work, div, burst_ms, local, peaks, seconds):
    """The same step back to back for >= `seconds` (no gaps, no host sync inside): long enough for
    the power cap to pull the SM clock to its sustained value and for nvidia-smi to see it."""
    n = max(10, int(seconds * 1e3 / max(burst_ms, 1e-3) * 1.15) + 1)
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.15)
    torch.cuda.synchronize()
    s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    s_ev.record()
    for _ in range(n):
        step()
    e_ev.record()
    torch.cuda.synchronize()
    t1 = time.time()
    clocks = sampler.stop(t0, t1)
    ms = s_ev.elapsed_time(e_ev) / n
    rate = work / (ms * 1e-3) / div
    out = {"steps": n, "seconds": (t1 - t0), "ms_per_step": ms, "tflops": rate,
           "sm_mhz_median": clocks.get("sm_mhz"), "power_w": clocks.get("power_w"),
           "samples_in_region": clocks.get("samples_in_timed_region"), "reasons": clocks.get("reasons")}
    if peaks.get("bf16_sustained"):
        out["frac"] = rate / peaks["bf16_sustained"]
        out["peak"] = peaks["bf16_sustained"]
        out["peak_source"] = f"{peaks['source']} cuBLAS bf16 sustained"
    if clocks.get("sm_mhz"):
        out["tflops_per_ghz"] = rate / (clocks["sm_mhz"] / 1e3)
    return out


def also_fp8_block(sizes, sizes_dev, dev, rank, peaks, steps, warmup):
    """The other half of the metric: the block-scaled FP8 gate+up GEMM (K=4096, N=3072) on the same
    routing, device-timed, with a parity figure taken inside the run: for EVERY group 8 rows (first,
    middle, last) x the first and last 128 output columns against the CPU oracle."""
    import oracle as O

    name = "fp8_block_m_grouped_gate_up"
    kind, k, n, trans_b = WORKLOADS[name]
    inp = make_inputs(kind, k, n, trans_b, sizes, dev, seed=300 + rank)
    step, _ = build_step(kind, k, n, trans_b, sizes_dev, inp)
    per = timed_steps(step, steps, max(warmup, 3))
    work, _ = algorithmic_work(kind, k, n, sizes)
    mean_ms = statistics.mean(per)
    rate = work / (mean_ms * 1e-3) / 1e12
    starts = (torch.cumsum(sizes, 0) - sizes).tolist()
    num = den = 0.0
    checked = 0
    cols = [(0, 128), (n - 128, n)]
    for g, (s0, sz) in enumerate(zip(starts, sizes.tolist())):
        if sz <= 0:
            continue
        pick = sorted({0, 1, 2, sz // 2, sz // 2 + 1, sz - 3, sz - 2, sz - 1} & set(range(sz)))
        rows = torch.tensor([s0 + r for r in pick], device=dev)
        a8, a_s, got = inp["a8"][rows].cpu(), inp["a_s"][rows].cpu(), inp["c"][rows].cpu().float()
        for c0, c1 in cols:
            ref = O.fp8_block_m_grouped_ref(a8, a_s, inp["b8"][g:g + 1, c0:c1].cpu(),
                                            inp["b_s"][g:g + 1, c0 // 128:c1 // 128].cpu(), [len(pick)]).float()
            num += float((got[:, c0:c1] - ref).abs().sum())
            den += float(ref.abs().sum())
        checked += 1
    peak = 2.0 * peaks["bf16"]
    return {"workload": name, "K": k, "N": n, "dtype": "fp8_e4m3", "steps": steps, "ms_per_step": mean_ms,
            "min_ms": min(per), "value": rate, "unit": "TFLOP/s",
            "roofline": {"bound": "tensor", "achieved": rate, "peak": peak, "frac": rate / peak,
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst x2 (no fp8 peak measured)",
                         "frac_of_nominal": rate / 4500.0},
            "parity": {"rdiff_vs_oracle": num / max(den, 1e-30), "groups_checked": checked, "rows_per_group": 8,
                       "columns": "first and last 128", "tolerance": 2e-3}}


REFERENCE_GPU_CHILD = r"""
import json, sys, torch
sys.path.insert(0, sys.argv[1])
sizes = json.loads(sys.argv[2]); k = int(sys.argv[3]); n = int(sys.argv[4]); scale = float(sys.argv[5])
from gemm.BF16.m_grouped_gemm_TMA import _build_m_grouped_metadata, _m_grouped_gemm_launch
dev = torch.device('cuda', 0)
gen = torch.Generator(device=dev).manual_seed(100)
sz = torch.tensor(sizes, device=dev, dtype=torch.int64)
m = int(sum(sizes))
a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
for r in range(0, m, 65536):
    rows = min(65536, m - r)
    a[r:r + rows] = (torch.randn(rows, k, device=dev, generator=gen) * scale).bfloat16()
b = (torch.randn(len(sizes), n, k, device=dev, generator=gen) * scale).bfloat16()
c = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
meta = _build_m_grouped_metadata(sz)
fn = lambda: _m_grouped_gemm_launch(a, b, c, sz, True, -1, metadata=meta, use_fixed_sm90_config=False)
for _ in range(5):
    fn()
torch.cuda.synchronize()
ts = []
for _ in range(10):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(); fn(); e.record(); e.synchronize()
    ts.append(s.elapsed_time(e))
g0 = sizes[0]
ref = (a[:min(g0, 256)].float() @ b[0].float().t())
err = ((c[:min(g0, 256)].float() - ref).abs().sum() / ref.abs().sum()).item()
print('REFJSON ' + json.dumps({'min_ms': min(ts), 'mean_ms': sum(ts) / len(ts), 'rdiff_group0_vs_fp32': err}))
"""


def gpu_reference_leg(sizes, k, n, work):
    """The reference's own Triton kernel (unmodified, autotuned) on the same sizes and data
    distribution, in a child process (its module registers the same torch operator name as this
    package, so the two cannot share an interpreter), metadata prebuilt as in its benchmark main."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "gemm" / "BF16" / "m_grouped_gemm_TMA.py").exists():
        return {"unavailable": "no installed copy of the reference under baseline/_ref"}
    try:
        r = subprocess.run([sys.executable, "-c", REFERENCE_GPU_CHILD, str(ref_root), json.dumps([int(v) for v in sizes.tolist()]),
                            str(k), str(n), str(DATA_SCALE[0])], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                           text=True, timeout=420)
    except Exception as exc:  # timeout, missing interpreter
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    for line in r.stdout.splitlines():
        if line.startswith("REFJSON "):
            d = json.loads(line[8:])
            d.update(impl="reference Triton kernel m_grouped_gemm_bKmajor_kernel (baseline/_ref), autotuned; 5 warm-ups, 10 timed",
                     value=work / (d["mean_ms"] * 1e-3) / 1e12, value_min_time=work / (d["min_ms"] * 1e-3) / 1e12,
                     unit="TFLOP/s")
            return d
    return {"unavailable": ("rc=%d: " % r.returncode + (r.stderr or r.stdout)[-300:]).replace("\n", " | ")}


def summarise_phases(marks, chunks):
    """[(phase, ms since start)] of one traced step -> per-chunk durations and the exposed head / tail."""
    t = dict(marks)
    out = {"plan_ms": t.get("plan_done", 0.0),
           "head_ms_until_first_gemm": t.get("gemm0>", 0.0), "step_ms": t.get("end", 0.0),
           "tail_ms_after_last_gemm": t.get("end", 0.0) - t.get(f"gemm{chunks - 1}<", 0.0),
           "final_combine_ms": t.get("end", 0.0) - t.get("returned_everywhere", 0.0)}
    for name in ("dispatch", "gemm", "return"):
        out[name + "_ms"] = [round(t[f"{name}{c}<"] - t[f"{name}{c}>"], 3) for c in range(chunks) if f"{name}{c}<" in t]
    out["gemm_wait_ms"] = [round(t[f"gemm{c}>"] - (t[f"gemm{c - 1}<"] if c else t.get("plan_done", 0.0)), 3)
                           for c in range(chunks) if f"gemm{c}>" in t]
    return out


def ep_leg(dev, rank, world, steps, warmup, chunks, comm_sms, qod=False, return_path="copy", transports=("p2p", "nccl"),
           taper=False, dispatch_path="kernel", ret_streams=2):
    """The expert-parallel FP8 MoE layer of the benchmark configuration on this process group:
    128 experts split over the ranks, 81 920 tokens x hidden 4096 per rank, top-8, intermediate
    1536; dispatch and combine over NVLink inside every step.  Both transports are timed (max over
    ranks); `gemm_only_ms` is the same rank's expert GEMMs + SwiGLU quantiser on the rows it
    received, with no exchange and every SM.  Each transport's result is first compared with the
    single-rank layer on a small step (must be identical).  Ends with the masked decode step."""
    import torch.distributed as dist

    from triton_grouped_gemm_b200 import _lib
    from triton_grouped_gemm_b200.ep.moe_layer import Fp8MoELayer, synthetic_routing

    group = dist.group.WORLD
    hidden, inter, tokens = 4096, 1536, 81920
    e_loc = NUM_EXPERTS // world
    res = {"tokens_per_rank": tokens, "top_k": TOP_K, "hidden": hidden, "intermediate": inter,
           "experts_per_rank": e_loc, "steps": steps, "transports": {}}

    def max_over_ranks(v):
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---- parity: a small layer against the single-rank layer, per transport (as the 2-GPU test does)
    se, sh, si, sk, st = 32, 512, 256, 4, 1024
    g0 = torch.Generator().manual_seed(0)
    sw13 = (torch.randn(se, 2 * si, sh, generator=g0) * 0.05).bfloat16()
    sw2 = (torch.randn(se, sh, si, generator=g0) * 0.05).bfloat16()
    sl = se // world
    full = Fp8MoELayer(sw13.to(dev), sw2.to(dev), se, None)
    sx = torch.randn(st, sh, generator=torch.Generator().manual_seed(100 + rank)).bfloat16().to(dev)
    sidx, sw = synthetic_routing(st, se, sk, seed=200 + rank, device=dev)
    ref = full.forward(sx, sidx, sw)
    small_rdiff = {}
    for transport, ch in [tc for tc in (("p2p", min(chunks, sl)), ("nccl", min(4, sl))) if tc[0] in transports]:
        lay = Fp8MoELayer(sw13[rank * sl:(rank + 1) * sl].to(dev), sw2[rank * sl:(rank + 1) * sl].to(dev), se, group,
                          transport=transport, chunks=ch, tokens_per_rank=st, top_k=sk, capacity_factor=2.0,
                          quantise_on_dispatch=qod, return_path=return_path, dispatch_path=dispatch_path,
                          ret_streams=ret_streams)
        out = lay.forward(sx, sidx, sw)
        small_rdiff[transport] = max_over_ranks(((out.float() - ref.float()).abs().sum() / ref.float().abs().sum()).item())
        lay.close()
    del full

    # ---- the benchmark-size layer
    gen = torch.Generator(device=dev).manual_seed(700 + rank)

    def randn(shape, scale):
        out = torch.empty(shape, device=dev, dtype=torch.bfloat16)
        for i in range(shape[0]):
            out[i] = (torch.randn(shape[1:], device=dev, generator=gen) * scale).bfloat16()
        return out

    w13, w2 = randn((e_loc, 2 * inter, hidden), 0.02), randn((e_loc, hidden, inter), 0.02)
    x = torch.randn(tokens, hidden, device=dev, generator=gen, dtype=torch.bfloat16)
    idx, w = synthetic_routing(tokens, NUM_EXPERTS, TOP_K, seed=ROUTING_SEED + rank, device=dev)
    work_rank = 2.0 * tokens * TOP_K * (2 * inter * hidden + hidden * inter)
    for transport, ch in [tc for tc in (("p2p", chunks), ("nccl", 4)) if tc[0] in transports]:
        layer = Fp8MoELayer(w13, w2, NUM_EXPERTS, group, chunks=ch, comm_sms=comm_sms, transport=transport,
                            tokens_per_rank=tokens, top_k=TOP_K, quantise_on_dispatch=qod, return_path=return_path, taper=taper,
                            dispatch_path=dispatch_path, ret_streams=ret_streams)
        dist.barrier()
        per = timed_steps(lambda: layer.forward(x, idx, w), steps, max(warmup, 3))
        ms = max_over_ranks(statistics.mean(per))
        entry = {"chunks": layer.chunks, "comm_sms": layer.comm_sms, "quantise_on_dispatch": bool(qod and transport == "p2p"),
                 "return_path": return_path if transport == "p2p" else "all_to_all",
                 "dispatch_path": layer.dispatch_path if transport == "p2p" else "all_to_all",
                 "return_queues": 1 + len(getattr(layer, "_ret_extra", [])) if transport == "p2p" else 0,
                 "ms_per_step": ms,
                 "tflops": work_rank * world / (ms * 1e-3) / 1e12, "rdiff_vs_single_rank": small_rdiff[transport]}
        if transport == "p2p":
            # the same rows without any exchange: this rank's expert GEMMs + SwiGLU quantiser, all SMs
            rows, sizes = layer.last_rows
            a8 = layer.recv8.local[:rows].view(torch.float8_e4m3fn)
            per_g = timed_steps(lambda: layer.experts(a8, layer.recvs.local[:rows], sizes, out=layer.ybuf.local[:rows]),
                                steps, 3)
            gemm_ms = max_over_ranks(statistics.mean(per_g))
            entry.update(gemm_only_ms=gemm_ms, efficiency=gemm_ms / ms, exposed_comm_ms=ms - gemm_ms,
                         rows_received_rank0=int(rows))
            if layer.chunks > 1:
                # one more step with CUDA events around every phase (rank 0's view)
                layer.trace = True
                dist.barrier()
                layer.forward(x, idx, w)
                entry["phases_rank0"] = summarise_phases(layer.phase_times(), layer.chunks)
                layer.trace = False
        st_word = torch.tensor([_lib.device_status()], device=dev, dtype=torch.int64)
        dist.all_reduce(st_word, op=dist.ReduceOp.MAX)
        entry["device_status"] = int(st_word[0])
        res["transports"][transport] = entry
        if transport == "p2p":
            res.update(ms_per_step=ms, tflops=entry["tflops"], gemm_only_ms=entry["gemm_only_ms"],
                       efficiency=entry["efficiency"], exposed_comm_ms=entry["exposed_comm_ms"],
                       rdiff_vs_single_rank=entry["rdiff_vs_single_rank"], device_status=entry["device_status"],
                       transport="p2p")
            # ---- decode: masked layout [experts per rank, 256 slots, hidden], valid counts uniform in [0, 256]
            from triton_grouped_gemm_b200.quant.per_block_cast import per_token_cast_to_fp8

            masked = torch.randint(0, DECODE_M_MAX + 1, (e_loc,), generator=torch.Generator().manual_seed(ROUTING_SEED + rank),
                                   dtype=torch.int64)
            xd = torch.randn(e_loc * DECODE_M_MAX, hidden, device=dev, generator=gen, dtype=torch.bfloat16)
            x8, xs = per_token_cast_to_fp8(xd)
            outd = torch.zeros(e_loc * DECODE_M_MAX, hidden, device=dev, dtype=torch.bfloat16)
            md = masked.to(dev)
            per_d = timed_steps(lambda: layer.decode(x8, xs, md, DECODE_M_MAX, out=outd), max(steps, 10), 3)
            dms = max_over_ranks(statistics.mean(per_d))
            valid = torch.tensor([float(masked.sum())], device=dev, dtype=torch.float64)
            dist.all_reduce(valid)
            res["decode"] = {"layout": [e_loc, DECODE_M_MAX, hidden], "ms_per_step": dms,
                             "valid_rows_all_ranks": int(valid[0]),
                             "tflops": 2.0 * float(valid[0]) * (2 * inter * hidden + hidden * inter) / (dms * 1e-3) / 1e12,
                             "weights_gb_per_rank": e_loc * 3 * inter * hidden / 1e9,
                             "note": "bound by streaming the expert weights (fp8) from HBM, not by the tensor cores"}
        layer.close()
        del layer
    return res


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    use_all_host_threads()  # the other ranks have exited: this is the only CPU work of the job
    kind, k, n, trans_b = WORKLOADS[args.workload]
    sizes = (moe_sizes(kind, max(args.gpus, 1), 0, args.rows) if kind in ("moe_ep", "moe_decode")
             else rank_sizes(max(args.gpus, 1), 0, args.rows, args.experts))
    unit, div = unit_of(kind)
    budget = 0.6e12 if unit == "TFLOP/s" else 1.5e9
    fn, work, desc = cpu_reference_step(kind, k, n, trans_b, sizes, budget)
    for _ in range(max(args.warmup, 1)):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = (time.perf_counter() - t0) / args.steps
    value = work / dt / div
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": metric_name(kind), "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dtype_name(kind), "data": "synthetic",
        "config": config_of(args.workload, kind, k, n, trans_b, sizes, args.gpus),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": desc,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(kind):
    return {"m_grouped": "grouped-GEMM TFLOP/s (BF16 M-grouped)", "k_grouped": "grouped-GEMM TFLOP/s (BF16 K-grouped)",
            "fp8_block": "grouped-GEMM TFLOP/s (FP8 block-scaled M-grouped)",
            "fp8_rowcol": "grouped-GEMM TFLOP/s (FP8 row x channel scales, M-grouped)",
            "fp8_rowcol_k": "grouped-GEMM TFLOP/s (FP8 row x channel scales, K-grouped)",
            "fp8_block_k": "grouped-GEMM TFLOP/s (FP8 block-scaled K-grouped, weight gradient)",
            "masked": "grouped-GEMM TFLOP/s (BF16 masked M-grouped)",
            "quant_act": "per-block quantiser GB/s (1x128 e4m3)",
            "quant_permute": "per-block quantiser + token permute GB/s (1x128 e4m3, top-8)",
            "quant_trans": "per-block quantiser GB/s (transposing 128x128 e4m3 with expansion)",
            "moe_ep": "expert-parallel FP8 MoE layer, grouped-GEMM TFLOP/s incl. dispatch/combine",
            "moe_decode": "FP8 MoE decode (masked layout), grouped-GEMM TFLOP/s"}[kind]


def dtype_name(kind):
    return {"m_grouped": "bf16", "k_grouped": "bf16", "fp8_block": "fp8_e4m3", "fp8_rowcol": "fp8_e4m3",
            "fp8_rowcol_k": "fp8_e4m3", "fp8_block_k": "fp8_e4m3", "masked": "bf16", "quant_act": "bf16->fp8_e4m3",
            "quant_permute": "bf16->fp8_e4m3",
            "quant_trans": "bf16->fp8_e4m3", "moe_ep": "fp8_e4m3", "moe_decode": "fp8_e4m3"}[kind]


def config_of(name, kind, k, n, trans_b, sizes, gpus):
    if kind == "moe_ep" and gpus > 1:
        partition = (f"experts split {NUM_EXPERTS}/{gpus} per GPU; every step dispatches fp8 rows to the expert owners and "
                     f"returns bf16 results over NVLink (transport {EP_TRANSPORT}, {EP_CHUNKS} chunks)")
    elif kind in ("moe_ep", "moe_decode"):
        partition = f"experts split {NUM_EXPERTS}/{gpus} per GPU; no exchange in this workload at this GPU count"
    else:
        partition = f"experts split {NUM_EXPERTS}/{gpus} per GPU, no data-path collective"
    return {"workload": name, "groups_per_gpu": int(sizes.numel()), "routed_rows_per_gpu": int(ROWS_USED[0]),
            "padded_rows_rank0": int(sizes.sum()), "K": k, "N": n, "trans_b": trans_b, "partition": partition,
            "l2": "inputs (>2.7 GB per step) exceed the 126 MB L2; no explicit flush"}


def run_b200(args):
    rank, world, local = dist_env()
    if world != max(args.gpus, 1):
        # launched without torchrun but with --gpus N>1: only rank 0's share can run here
        if world == 1 and args.gpus > 1:
            print(json.dumps({"error": "launch with torch.distributed.run for --gpus > 1"}), flush=True)
            return 2
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    from triton_grouped_gemm_b200 import _lib

    _lib.load()
    if args.ep_only and use_dist:
        ep = ep_leg(dev, rank, world, min(args.steps, 8), 3, args.ep_chunks, args.ep_comm_sms, args.ep_quantise_on_dispatch, args.ep_return_path,
                    transports=("p2p",) if args.ep_skip_nccl else ("p2p", "nccl"), taper=args.ep_taper,
                    dispatch_path=args.ep_dispatch_path, ret_streams=args.ep_ret_streams)
        if rank == 0:
            print(json.dumps({"ep_only": True, "n_gpus": world, "ep": ep}), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return 0
    kind, k, n, trans_b = WORKLOADS[args.workload]
    if args.workload in UNIFORM_WORKLOADS:
        UNIFORM[0] = True
        DATA_SCALE[0] = 1.0
    sizes = (moe_sizes(kind, world, rank, args.rows) if kind in ("moe_ep", "moe_decode")
             else rank_sizes(world, rank, args.rows, args.experts))
    if kind == "masked":  # valid rows per 4096-row slot, ~1/4 full, every fifth slot empty
        gen_m = torch.Generator().manual_seed(ROUTING_SEED + rank)
        sizes = torch.randint(0, 2049, (sizes.numel(),), generator=gen_m, dtype=torch.int64)
        sizes[::5] = 0
    sizes_dev = sizes.to(dev)
    global EP_CHUNKS, EP_TRANSPORT, EP_COMM_SMS
    EP_CHUNKS = args.ep_chunks
    EP_TRANSPORT = args.ep_transport
    EP_COMM_SMS = args.ep_comm_sms
    if args.cta_pair != -1:
        from triton_grouped_gemm_b200 import _lib

        _lib.load().b200gemm_set_cta_pair(args.cta_pair)
    inp = make_inputs(kind, k, n, trans_b, sizes, dev, seed=100 + rank)
    step, launches = build_step(kind, k, n, trans_b, sizes_dev, inp)
    work, _ = algorithmic_work(kind, k, n, sizes)
    if kind == "moe_ep":
        work = 2.0 * (args.rows // TOP_K) * TOP_K * (2 * n * k + k * n)
    unit, div = unit_of(kind)

    def barrier():
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = args.warmup if args.profile else max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)
    # ---- device-timed region: exactly `steps` steps, one CUDA event pair per step
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    t_epoch_begin = time.time()
    t_wall = time.perf_counter()
    for s_ev, e_ev in evs:
        s_ev.record()
        step()
        e_ev.record()
    barrier()
    t_wall = time.perf_counter() - t_wall
    per_step = [s.elapsed_time(e) for s, e in evs]
    total_ms = evs[0][0].elapsed_time(evs[-1][1])
    clocks = sampler.stop(t_epoch_begin, t_epoch_begin + t_wall) if sampler else None
    status = _lib.device_status()
    if status:
        raise RuntimeError(f"device status word = {status:#x} (a bounded wait ran out)")

    tot = torch.tensor([total_ms, work], device=dev, dtype=torch.float64)
    if use_dist:
        mx = tot.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = tot.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms_max, work_all = float(mx[0]), float(sm[1])
    else:
        total_ms_max, work_all = total_ms, work
    ms_per_step = total_ms_max / args.steps
    value = work_all / (ms_per_step * 1e-3) / div
    extras = not (args.no_extras or args.profile)
    sustained = None
    if extras and args.sustain_seconds > 0 and kind not in ("moe_ep", "moe_decode"):
        barrier()
        sustained = sustained_leg(step, work, div, statistics.mean(per_step), local, measured_peaks(), args.sustain_seconds)
        barrier()

    # ---- end to end through the public operator with host (pinned) buffers
    if args.profile:
        # profiling run (under ncu): device-timed steps only, no host-buffer leg, no CPU leg
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": args.workload, "ms_per_step": ms_per_step,
                              "value": value, "unit": unit, "rows": int(sizes.sum()), "groups": int(sizes.numel())}),
                  flush=True)
        if use_dist:
            dist.barrier()
            dist.destroy_process_group()
        return 0
    e2e = run_e2e(args, kind, k, n, trans_b, sizes, inp, dev, use_dist, work_all if not use_dist else None, work)
    if use_dist:
        t = torch.tensor([e2e["ms"]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e["ms"] = float(t[0])
        e2e_value = work_all / (e2e["ms"] * 1e-3) / div
    else:
        e2e_value = work / (e2e["ms"] * 1e-3) / div

    if rank == 0:
        peaks = measured_peaks()
        # a multi-kernel step (MoE layer) is judged as a whole: flops of its GEMMs over the step time
        launch_ms = statistics.mean(per_step) / (1 if kind in ("moe_ep", "moe_decode") else launches)
        if unit == "TFLOP/s":
            fp8 = kind in ("fp8_block", "moe_ep", "moe_decode", "fp8_rowcol", "fp8_rowcol_k", "fp8_block_k")
            peak = peaks["bf16"] * (2.0 if fp8 else 1.0)
            achieved = work / (launch_ms * 1e-3) / 1e12
            # DRAM bytes per launch from the ncu capture of the 82 560-row case of this kernel
            # (668.7 MB: 569 MB scale with rows, 100 MB with experts), scaled to this launch
            traffic = None
            if args.workload == "bf16_m_grouped_gate_up":
                traffic = 568.9e6 * int(sizes.sum()) / 82560.0 + 99.8e6 * sizes.numel() / 16.0
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": traffic,
                    "peak_source": f"{peaks['source']} cuBLAS bf16 burst" + (" x2 (no fp8 peak measured)" if fp8 else ""),
                    "frac_of_nominal": achieved / (4500.0 if fp8 else 2250.0),
                    "min_ms": min(per_step), "mean_ms": statistics.mean(per_step)}
        else:
            achieved = work / (launch_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm"], "traffic": None, "peak_source": f"{peaks['source']} copy",
                    "min_ms": min(per_step), "mean_ms": statistics.mean(per_step)}
        cpu = None
        if not args.no_cpu_baseline:
            use_all_host_threads()  # under torchrun OMP_NUM_THREADS is 1; the other ranks idle at a barrier meanwhile
            fn, cwork, desc = cpu_reference_step(kind, k, n, trans_b, sizes, 0.6e12 if unit == "TFLOP/s" else 1.5e9)
            fn()
            best = float("inf")
            t_begin = time.perf_counter()
            reps = 0
            while reps < 3 or (time.perf_counter() - t_begin < 10 and reps < 20):
                t0 = time.perf_counter()
                fn()
                best = min(best, time.perf_counter() - t0)
                reps += 1
            cpu = {"value": cwork / best / div, "unit": unit, "cores": torch.get_num_threads(), "kind": "port",
                   "sample": desc + f"; best of {reps}", "host_cpus": os.cpu_count()}
        line = {
            "metric": metric_name(kind), "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype_name(kind), "data": "synthetic",
            "config": config_of(args.workload, kind, k, n, trans_b, sizes, world),
            "roofline": roof, "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                    "steps": e2e["steps"], "ms_per_step": e2e["ms"]},
            "gpu_launches": launches * args.steps, "clocks": clocks, "wall_s_timed_region": t_wall,
        }
        if sustained is not None and unit == "TFLOP/s":
            line["roofline"]["sustained"] = sustained
        elif sustained is not None:
            sustained["gbs"] = sustained.pop("tflops")
            sustained.pop("frac", None), sustained.pop("peak", None), sustained.pop("peak_source", None)
            sustained.pop("tflops_per_ghz", None)
            line["roofline"]["sustained"] = sustained
    # ---- the rest of the metric, measured in the same run
    also = gpu_ref = ep = None
    layer = inp.get("layer")
    if extras and args.workload == "bf16_m_grouped_gate_up":
        inp.clear()
        step = None  # the closure holds the operands
        torch.cuda.empty_cache()
        if use_dist:
            dist.barrier()
        also = also_fp8_block(sizes, sizes_dev, dev, rank, measured_peaks(), min(args.steps, 10), 3)
        torch.cuda.empty_cache()
        if not use_dist and rank == 0:
            gpu_ref = gpu_reference_leg(sizes, k, n, work)
        if use_dist:
            dist.barrier()
            ep = ep_leg(dev, rank, world, min(args.steps, 8), 3, args.ep_chunks, args.ep_comm_sms,
                        args.ep_quantise_on_dispatch, args.ep_return_path, dispatch_path=args.ep_dispatch_path,
                        ret_streams=args.ep_ret_streams)
    if rank == 0:
        if also is not None:
            line["also"] = also
        if gpu_ref is not None:
            line["gpu_reference"] = gpu_ref
            if "value" in gpu_ref:
                line["gpu_reference"]["this_build_over_reference"] = value / gpu_ref["value"]
        if ep is not None:
            line["ep"] = ep
        print(json.dumps(line), flush=True)
    if layer is not None:
        layer.close()  # collective; releases the peer-memory buffers before the process group goes away
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_e2e(args, kind, k, n, trans_b, sizes, inp, dev, use_dist, _unused, work):
    """Host inputs (pinned) -> device -> operator -> host result, every step."""
    steps = max(1, min(args.steps, args.e2e_steps))
    if kind == "m_grouped":
        # the library's host-operand entry point: chunked H2D / GEMM / D2H pipeline on three streams
        from triton_grouped_gemm_b200.host import m_grouped_gemm_host

        host = {"a": inp["a"].cpu().pin_memory(), "b": inp["b"].cpu().pin_memory(), "s": sizes.pin_memory()}
        out_host = torch.empty(inp["a"].shape[0], n, dtype=torch.bfloat16).pin_memory()
        del inp["c"], inp["a"], inp["b"]

        def one():
            m_grouped_gemm_host(host["a"], host["b"], host["s"], trans_b, out_host=out_host, device=dev)
    elif kind == "k_grouped":
        from triton_grouped_gemm_b200.gemm.BF16.k_grouped_gemm_TMA import k_grouped_gemm

        host = {"a": inp["a"].cpu().pin_memory(), "b": inp["b"].cpu().pin_memory(), "s": sizes.pin_memory()}
        out_host = torch.empty(sizes.numel(), k, n, dtype=torch.bfloat16).pin_memory()

        def one():
            a = host["a"].to(dev, non_blocking=True)
            b = host["b"].to(dev, non_blocking=True)
            s = host["s"].to(dev, non_blocking=True)
            out_host.copy_(k_grouped_gemm(a, b, s), non_blocking=True)
    elif kind == "fp8_block":
        from triton_grouped_gemm_b200.gemm.FP8.m_grouped_gemm_block_scaled import m_grouped_fp8_block_scaled

        host = {kk: inp[kk].cpu().pin_memory() for kk in ("a8", "a_s", "b8", "b_s")}
        host["s"] = sizes.pin_memory()
        out_host = torch.empty(inp["a8"].shape[0], n, dtype=torch.bfloat16).pin_memory()
        del inp["c"]

        def one():
            d = {kk: v.to(dev, non_blocking=True) for kk, v in host.items()}
            c = m_grouped_fp8_block_scaled((d["a8"], d["a_s"]), (d["b8"], d["b_s"]), d["s"])
            out_host.copy_(c, non_blocking=True)
    elif kind in ("fp8_rowcol", "fp8_rowcol_k", "masked", "fp8_block_k"):
        # generic: every operand from pinned host memory, the operator, the result back to the host
        names = [kk for kk, v in inp.items() if isinstance(v, torch.Tensor) and kk != "c"]
        # scale matrices of the K-grouped workload are transposed views of group-major memory
        transposed = {kk for kk in names if not inp[kk].is_contiguous()}
        host = {kk: (inp[kk].t().contiguous() if kk in transposed else inp[kk]).cpu().pin_memory() for kk in names}
        host["s"] = sizes.pin_memory()
        out_host = torch.empty(inp["c"].shape, dtype=inp["c"].dtype).pin_memory()
        for kk in names + ["c"]:
            del inp[kk]

        def one():
            d = {}
            for kk in names:
                t = host[kk].to(dev, non_blocking=True)
                d[kk] = t.t() if kk in transposed else t
            fn, _ = build_step(kind, k, n, trans_b, host["s"].to(dev, non_blocking=True), d)
            fn()
            out_host.copy_(d["c"], non_blocking=True)
    elif kind == "moe_ep":
        layer = inp["layer"]
        host = {"x": inp["x"].cpu().pin_memory(), "idx": inp["idx"].cpu().pin_memory(), "w": inp["w"].cpu().pin_memory()}
        out_host = torch.empty(inp["x"].shape, dtype=torch.bfloat16).pin_memory()

        def one():
            d = {kk: v.to(dev, non_blocking=True) for kk, v in host.items()}
            out_host.copy_(layer.forward(d["x"], d["idx"], d["w"]), non_blocking=True)
    elif kind == "moe_decode":
        layer = inp["layer"]
        host = {"x8": inp["x8"].cpu().pin_memory(), "xs": inp["xs"].cpu().pin_memory(), "s": sizes.pin_memory()}
        out_host = torch.empty(inp["out"].shape, dtype=torch.bfloat16).pin_memory()

        def one():
            d = {kk: v.to(dev, non_blocking=True) for kk, v in host.items()}
            out_host.copy_(layer.decode(d["x8"], d["xs"], d["s"], DECODE_M_MAX), non_blocking=True)
    elif kind == "quant_trans":
        from triton_grouped_gemm_b200.quant.trans_per_block_quant_expand_128x import trans_per_block_quant_expand_128x

        host = {"x": inp["x"].cpu().pin_memory(), "s": sizes.pin_memory()}
        q0, s0, _ = inp["c"]
        out_host = torch.empty(q0.shape, dtype=torch.uint8).pin_memory()
        s_host = torch.empty(s0.shape, dtype=torch.float32).pin_memory()

        def one():
            q, sc, _ = trans_per_block_quant_expand_128x(host["x"].to(dev, non_blocking=True),
                                                         host["s"].to(dev, non_blocking=True))
            out_host.copy_(q.view(torch.uint8), non_blocking=True)
            s_host.copy_(sc, non_blocking=True)
        host["_extra_out"] = s_host
    elif kind == "quant_permute":
        from triton_grouped_gemm_b200.ep.dispatch import quant_permute_rows

        host = {"x": inp["x"].cpu().pin_memory(), "pos": inp["pos"].cpu().pin_memory()}
        q0, s0 = inp["c"]
        out_host = torch.empty(q0.shape, dtype=torch.uint8).pin_memory()
        s_host = torch.empty(s0.shape, dtype=torch.float32).pin_memory()

        def one():
            q, sc = quant_permute_rows(host["x"].to(dev, non_blocking=True), host["pos"].to(dev, non_blocking=True), TOP_K)
            out_host.copy_(q.view(torch.uint8), non_blocking=True)
            s_host.copy_(sc, non_blocking=True)
        host["_extra_out"] = s_host
    else:
        from triton_grouped_gemm_b200.quant.per_block_cast import per_token_cast_to_fp8

        host = {"x": inp["x"].cpu().pin_memory()}
        q_host = torch.empty(inp["x"].shape, dtype=torch.float8_e4m3fn).pin_memory()
        s_host = torch.empty(inp["x"].shape[0], k // 128, dtype=torch.float32).pin_memory()
        out_host = q_host

        def one():
            q, s = per_token_cast_to_fp8(host["x"].to(dev, non_blocking=True))
            q_host.copy_(q, non_blocking=True)
            s_host.copy_(s, non_blocking=True)
        host["_extra_out"] = s_host
    h2d = sum(v.numel() * v.element_size() for kk, v in host.items() if not kk.startswith("_"))
    d2h = out_host.numel() * out_host.element_size() + sum(
        v.numel() * v.element_size() for kk, v in host.items() if kk.startswith("_"))
    one()
    torch.cuda.synchronize()
    if use_dist:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()
    s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s_ev.record()
    for _ in range(steps):
        one()
    e_ev.record()
    torch.cuda.synchronize()
    return {"ms": s_ev.elapsed_time(e_ev) / steps, "h2d": h2d, "d2h": d2h, "steps": steps}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="bf16_m_grouped_gate_up")
    ap.add_argument("--e2e-steps", type=int, default=3, help="steps of the host-buffer end-to-end timing")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--rows", type=int, default=TOTAL_ROWS, help="routed rows per GPU (default: the benchmark's 655360)")
    ap.add_argument("--experts", type=int, default=NUM_EXPERTS, help="experts over all GPUs (default 128)")
    ap.add_argument("--ep-chunks", type=int, default=None,
                    help="moe_ep_fp8 with more than one GPU: groups of local experts whose exchange overlaps the GEMMs "
                         "(default: 8, and 16 from 8 GPUs on, where the shorter last chunk shortens the exposed tail)")
    ap.add_argument("--ep-transport", choices=["p2p", "nccl"], default="p2p",
                    help="moe_ep_fp8 with more than one GPU: rows move by kernels over peer memory (p2p) or by "
                         "NCCL all-to-all (nccl)")
    ap.add_argument("--cta-pair", type=int, default=-1, choices=[-1, 0, 1],
                    help="kernel form: -1 chosen by problem size (default), 0 single-CTA tiles, 1 CTA pairs")
    ap.add_argument("--ep-comm-sms", type=int, default=None,
                    help="moe_ep_fp8 with more than one GPU: SMs the expert GEMMs leave to the row movers / collectives "
                         "(default: the layer's own, 12 with mover kernels, 2 when both ways go by copy engine)")
    ap.add_argument("--ep-ret-streams", type=int, default=2,
                    help="expert-parallel leg, peer memory: stream queues the copy-engine return is spread over")
    ap.add_argument("--ep-dispatch-path", choices=["copy", "kernel"], default="kernel",
                    help="expert-parallel leg, peer memory: rows travel to the experts by copy engine after a local gather, "
                         "or by the mover kernels beside the GEMMs")
    ap.add_argument("--ep-quantise-on-dispatch", action="store_true",
                    help="expert-parallel p2p transport: quantise each pair's bf16 row inside the dispatch kernel")
    ap.add_argument("--ep-return-path", choices=["copy", "kernel"], default="copy",
                    help="expert-parallel p2p transport: results go home by copy engine (copy) or by the mover kernel")
    ap.add_argument("--ep-taper", action="store_true", help="with --ep-only: short first and last expert run")
    ap.add_argument("--ep-skip-nccl", action="store_true", help="with --ep-only: time the p2p transport only")
    ap.add_argument("--ep-only", action="store_true",
                    help="with more than one GPU: run only the expert-parallel leg and print its JSON (tuning runs)")
    ap.add_argument("--sustain-seconds", type=float, default=2.0,
                    help="length of the back-to-back (sustained) leg after the timed steps; 0 = skip")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline measurement: no sustained leg, no FP8 / reference-kernel / expert-parallel legs")
    ap.add_argument("--profile", action="store_true",
                    help="for ncu captures: honour --warmup as given, skip the host-buffer and CPU legs")
    args = ap.parse_args()
    if args.ep_chunks is None:
        args.ep_chunks = 16 if int(os.environ.get("WORLD_SIZE", "1")) >= 8 else 8
    ROWS_USED[0] = args.rows
    if args.impl == "reference":
        run_reference(args)
        return 0
    return run_b200(args)


if __name__ == "__main__":
    sys.exit(main() or 0)
