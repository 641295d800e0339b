"""Seeded inputs of the FP8 row x channel GEMM fixture (``fp8_rowcol.pt``).

Shared by ``make_golden_gpu.py`` (which builds them with the reference's own casts and runs the
reference's Triton kernels on them) and by the tests (which rebuild them with ``oracle/``'s
casts and check the stored SHA-256 of every input before comparing outputs), so the fixture
holds only hashes and outputs.  ``casts`` maps "per_channel_cast_to_fp8" and
"per_expert_cast_to_fp8" to callables with the reference's signatures
(gemm/FP8/m_grouped_gemm_channel_expert.py:224-261).
"""

from __future__ import annotations

import hashlib

import torch

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2

# name: (rows per group, N, K, activation format, weight format, output dtype, one weight scale per expert)
M_CASES = {
    "one_tile_e4e4": ([128], 256, 128, E4, E4, torch.bfloat16, False),
    "ragged_e5e4_fp16": ([125, 0, 309, 3], 512, 256, E5, E4, torch.float16, False),
    "ragged_e4e4_ktail": ([300, 77], 256, 272, E4, E4, torch.bfloat16, False),
    # the reference test's shape family (tests/test_FP8/test_m_grouped_gemm_channel_expert.py:104-126:
    # ragged experts, e5m2 x e4m3, one scale per expert expanded to [G, N]), scaled down
    "test_family_e5e4": ([253, 259, 125, 131], 256, 384, E5, E4, torch.bfloat16, True),
}
# name: (tokens per group -- multiples of 128, data zero padded --, M, N, dtype_a, dtype_b); 1 = e4m3, 2 = e5m2
K_CASES = {
    "one_tile_e4e4": ([128], 128, 256, 1, 1),
    "ragged_e4e4": ([256, 0, 128, 512], 256, 256, 1, 1),
    "ragged_e5e4": ([384, 128, 0, 256], 128, 256, 2, 1),
}


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def m_case_inputs(name: str, casts) -> dict:
    """a8 [M, K], a_scale [M, 1], b8 [G, N, K], b_scale [G, N], sizes int32 [G]."""
    sizes, n, k, fa, fb, dt_out, per_expert = M_CASES[name]
    gen = torch.Generator().manual_seed(1000 + n + k + len(sizes))
    m, g = sum(sizes), len(sizes)
    k_pad = (k + 127) // 128 * 128
    x = torch.randn(m, k_pad, generator=gen).to(torch.bfloat16)
    a8, a_s = casts["per_channel_cast_to_fp8"](x, fa)
    w = torch.randn(g, n, k_pad, generator=gen).to(torch.bfloat16)
    if per_expert:
        b8, b_s = casts["per_expert_cast_to_fp8"](w, fb)
        b_s = b_s.view(-1, 1).repeat(1, n)
    else:
        # an independent scale per (expert, channel): what the kernel's indexing g*N+n allows
        per = [casts["per_channel_cast_to_fp8"](w[i], fb) for i in range(g)]
        b8 = torch.stack([q for q, _ in per])
        b_s = torch.stack([s.view(-1) for _, s in per])
    return {"sizes": torch.tensor(sizes, dtype=torch.int32), "n": n, "k": k, "fmt_a": fa, "fmt_b": fb,
            "dtype_out": dt_out, "a8": a8[:, :k].contiguous(), "a_scale": a_s.contiguous(),
            "b8": b8[:, :, :k].contiguous(), "b_scale": b_s.reshape(g, n).contiguous()}


def k_case_inputs(name: str, casts) -> dict:
    """x8 [M, K_tot], y8 [N, K_tot]; x_scale / y_scale logical [M, G] / [N, G] over group-major
    memory, built the way the reference's generator does
    (tests/test_FP8/test_k_grouped_gemm_channel_expert.py:68-98)."""
    tokens, m, n, da, db = K_CASES[name]
    gen = torch.Generator().manual_seed(2000 + m + n + len(tokens))
    fa, fb = (E4 if da == 1 else E5), (E4 if db == 1 else E5)
    xs_l, ys_l, x_l, y_l = [], [], [], []
    for t in tokens:
        # per expert [M, tokens] / [N, tokens] with one scale per row; an empty expert contributes
        # no columns but still has scales
        xe = torch.randn(m, max(t, 128), generator=gen).to(torch.bfloat16)
        ye = torch.randn(n, max(t, 128), generator=gen).to(torch.bfloat16)
        if t >= 128:  # the last 5 tokens of every expert are padding zeros, as in the generator
            xe[:, t - 5:] = 0
            ye[:, t - 5:] = 0
        xq, xsc = casts["per_channel_cast_to_fp8"](xe, fa)
        yq, ysc = casts["per_channel_cast_to_fp8"](ye, fb)
        x_l.append(xq[:, :t])
        y_l.append(yq[:, :t])
        xs_l.append(xsc)
        ys_l.append(ysc)
    x_scale = torch.cat(xs_l, -1).contiguous().transpose(0, 1).contiguous().transpose(0, 1)
    y_scale = torch.cat(ys_l, -1).contiguous().transpose(0, 1).contiguous().transpose(0, 1)
    return {"tokens": torch.tensor(tokens, dtype=torch.int32), "m": m, "n": n, "dtype_a": da, "dtype_b": db,
            "fmt_a": fa, "fmt_b": fb, "x8": torch.cat(x_l, -1).contiguous(), "y8": torch.cat(y_l, -1).contiguous(),
            "x_scale": x_scale, "y_scale": y_scale}


def input_hashes(inp: dict) -> dict:
    out = {}
    for key, v in inp.items():
        if isinstance(v, torch.Tensor):
            # hash the memory order of the transposed scale views through their contiguous parent
            out[key] = sha(v.t() if (v.dim() == 2 and not v.is_contiguous()) else v)
    return out
