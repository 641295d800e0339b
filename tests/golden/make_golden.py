"""Generate the golden fixtures in this directory from the reference itself.

Run where a checkout of DeepLink-org/Triton_Grouped_GEMM is available:

    python tests/golden/make_golden.py --reference /path/to/Triton_Grouped_GEMM

Importable reference functions are imported (``gemm.BF16.utils.gmm``,
``m_grouped_reference``, ``gmm_dw_reference``, ``gemm.layout.*``).  The torch
quantisers live under ``if __name__ == "__main__":`` in their files, so their
``def`` nodes are lifted out with ``ast`` and executed unchanged on CPU.  Only
torch CPU code of the reference runs here -- none of its Triton kernels.

The fixtures hold inputs and the reference's outputs (fp8 tensors as uint8
views).  ``tests/test_oracle_golden.py`` checks ``oracle/`` against them.
"""

from __future__ import annotations

import argparse
import ast
import hashlib
import sys
from pathlib import Path
from typing import Tuple

import torch

HERE = Path(__file__).resolve().parent


def lift_functions(path: Path, names):
    """Return {name: function} for ``def``s found anywhere in ``path`` (incl. under __main__)."""
    tree = ast.parse(path.read_text())
    wanted = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in names and node.name not in wanted:
            wanted[node.name] = node
    missing = set(names) - set(wanted)
    if missing:
        raise RuntimeError(f"{path}: functions not found: {sorted(missing)}")
    import triton  # the lifted code calls triton.cdiv

    ns = {"torch": torch, "triton": triton, "Tuple": Tuple}
    # keep source order so helpers are defined before their users
    for node in sorted(wanted.values(), key=lambda n: n.lineno):
        mod = ast.Module(body=[node], type_ignores=[])
        exec(compile(mod, str(path), "exec"), ns)
    return {n: ns[n] for n in names}


def u8(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8).clone()


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of DeepLink-org/Triton_Grouped_GEMM")
    args = ap.parse_args()
    ref = Path(args.reference)
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

    from gemm.BF16.utils import gmm, row_max_normalization  # noqa: E402
    from gemm.BF16.m_grouped_gemm_TMA import m_grouped_reference  # noqa: E402
    from gemm.BF16.k_grouped_gemm_TMA import gmm_dw_reference  # noqa: E402
    from gemm import layout as ref_layout  # noqa: E402
    from oracle.torch_oracle import config0_inputs  # input generator only

    fp8_file = ref / "gemm/FP8/m_grouped_gemm_channel_expert.py"
    casts = lift_functions(
        fp8_file,
        ["ceil_div", "per_token_cast_to_fp8", "per_channel_cast_to_fp8", "per_block_cast_to_fp8",
         "per_expert_cast_to_fp8"],
    )
    # the lifted functions call each other through their own namespace (ceil_div)
    quant_file = ref / "quant/trans_per_block_quant_expand_128x.py"
    tq = lift_functions(
        quant_file,
        ["to_fp8_saturated", "per_block_trans_quant_expand_per_expert", "per_block_trans_quant_expand_torch"],
    )

    torch.manual_seed(1234)

    # ---- layouts -----------------------------------------------------------
    lay = {}
    for name, sizes, bm in (("a", [3, 5, 0, 7], 4), ("b", [3, 5], 4), ("c", [130, 0, 1, 128, 257], 128)):
        t = torch.tensor(sizes, dtype=torch.int32)
        gl = ref_layout.make_grouped_layout(sizes, block_m=bm)
        lay[name] = {
            "sizes": sizes,
            "block_m": bm,
            "round_up": ref_layout.round_up_to_alignment(t, bm).tolist(),
            "starts": ref_layout.make_group_starts(t, padded=False, block_m=bm).tolist(),
            "starts_padded": ref_layout.make_group_starts(t, padded=True, block_m=bm).tolist(),
            "grouped_layout": ref_layout.make_deep_gemm_grouped_layout(sizes, block_m=bm).tolist(),
            "psum": ref_layout.make_deep_gemm_psum_layout(sizes, block_m=bm).tolist(),
            "gl_starts": gl.starts.tolist(),
            "gl_padded": gl.padded_sizes.tolist(),
            "total_m": int(gl.total_m),
            "total_padded_m": int(gl.total_padded_m),
        }
    torch.save(lay, HERE / "layout.pt")

    # ---- BF16 M-grouped ------------------------------------------------------
    mg = {}
    a, b, sizes = config0_inputs(0)
    mg["config0"] = {"sizes": sizes, "a_sha": sha(a), "b_sha": sha(b),
                     "out": m_grouped_reference(a, b, sizes, True)}
    sizes_s = torch.tensor([5, 0, 19, 128, 1], dtype=torch.int64)
    a = (torch.randn(int(sizes_s.sum()), 96) * 0.5).to(torch.bfloat16)
    b_nk = (torch.randn(5, 40, 96) * 0.5).to(torch.bfloat16)
    b_kn = b_nk.transpose(1, 2).contiguous()
    mg["small_nt"] = {"sizes": sizes_s, "a": a, "b": b_nk, "out": m_grouped_reference(a, b_nk, sizes_s, True)}
    mg["small_nn"] = {"sizes": sizes_s, "a": a, "b": b_kn, "out": gmm(a, b_kn, sizes_s, trans_b=False)}
    a16 = a.to(torch.float16)
    mg["small_nt_fp16"] = {"sizes": sizes_s, "a": a16, "b": b_nk.to(torch.float16),
                           "out": m_grouped_reference(a16, b_nk.to(torch.float16), sizes_s, True)}
    torch.save(mg, HERE / "m_grouped.pt")

    # ---- BF16 masked (reference check = full per-group product, compared on the masked rows;
    #      tests/test_BF16/test_m_grouped_gemm_masked_TMA.py:88-92) --------------------------
    g_, e_, k_, n_ = 3, 128, 64, 48
    lhs = (torch.randn(g_ * e_, k_) * 0.5).to(torch.bfloat16)
    rhs = (torch.randn(g_, n_, k_) * 0.5).to(torch.bfloat16)
    full = gmm(lhs, rhs, torch.full((g_,), e_, dtype=torch.int64), trans_b=True)
    torch.save({"lhs": lhs, "rhs": rhs, "expected_m": e_, "masked_m": torch.tensor([17, 0, 128]),
                "full": full, "full_rownorm": row_max_normalization(full.float())}, HERE / "masked.pt")

    # ---- BF16 K-grouped ------------------------------------------------------
    ks = torch.tensor([33, 0, 64, 7], dtype=torch.int64)
    ka = (torch.randn(int(ks.sum()), 48) * 0.5).to(torch.bfloat16)
    kb = (torch.randn(int(ks.sum()), 40) * 0.5).to(torch.bfloat16)
    kout = gmm_dw_reference(ka, kb, ks)
    kout[1] = 0  # the reference leaves C[g] of an empty group as `lhs.T @ rhs` of 0 rows == zeros
    torch.save({"sizes": ks, "a": ka, "b": kb, "out": kout}, HERE / "k_grouped.pt")

    # ---- quantisers ----------------------------------------------------------
    q = {}
    x = torch.randn(24, 384).to(torch.bfloat16)
    x[3, 128:256] = 0  # a block whose amax hits the 1e-4 clamp
    x[5, 0] = 300.0
    x[6, 7] = -1e-3
    xq, xs = casts["per_token_cast_to_fp8"](x)
    q["per_token"] = {"x": x, "q": u8(xq), "s": xs}
    w = (torch.randn(200, 300) * 0.02).to(torch.bfloat16)
    wq, ws = casts["per_block_cast_to_fp8"](w)
    q["per_block"] = {"x": w, "q": u8(wq), "s": ws}
    for name, dt in (("per_channel_e4m3", torch.float8_e4m3fn), ("per_channel_e5m2", torch.float8_e5m2)):
        cq, cs = casts["per_channel_cast_to_fp8"](x, dt)
        q[name] = {"x": x, "q": u8(cq), "s": cs}
    we = (torch.randn(3, 128, 256) * 0.02).to(torch.bfloat16)
    for name, dt in (("per_expert_e4m3", torch.float8_e4m3fn), ("per_expert_e5m2", torch.float8_e5m2)):
        eq, es = casts["per_expert_cast_to_fp8"](we, dt)
        q[name] = {"x": we, "q": u8(eq), "s": es}
    torch.save(q, HERE / "casts.pt")

    tqf = {}
    for name, sizes, n in (("equal", [128, 128, 128], 256), ("ragged", [130, 0, 1, 127, 256, 5], 128)):
        t = torch.tensor(sizes)
        xin = torch.randn(int(t.sum()), n).to(torch.bfloat16)
        oq, os_, pad = tq["per_block_trans_quant_expand_torch"](xin, t)
        tqf[name] = {"x": xin, "sizes": t, "q": u8(oq), "s": os_, "padded": pad}
    torch.save(tqf, HERE / "trans_quant.pt")

    for f in sorted(HERE.glob("*.pt")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
