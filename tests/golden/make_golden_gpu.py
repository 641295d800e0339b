"""Generate ``fp8_rowcol.pt`` by running the reference's own Triton kernels on a GPU.

Run on a machine with a CUDA GPU and a checkout (or installed copy) of
DeepLink-org/Triton_Grouped_GEMM:

    python tests/golden/make_golden_gpu.py --reference /path/to/root/holding/gemm --out tests/golden/fp8_rowcol.pt

The two FP8 GEMMs with per-row x per-channel scales exist in the reference only as Triton
kernels (no torch twin), so the CPU script ``make_golden.py`` cannot pin them.  This script
calls ``gmm_fp8_act_per_channel_w_per_expert``
(gemm/FP8/m_grouped_gemm_channel_expert.py:139-198) and ``matmul``
(gemm/FP8/k_grouped_gemm_channel_expert.py:143-181) unchanged, on small ragged problems whose
inputs are built on the CPU from a seeded generator with the reference's own casts (lifted out
of the ``__main__`` block of the M-grouped file), and stores a SHA-256 of every input and the kernels' outputs (the inputs are rebuilt from
the seed by ``fp8_rowcol_cases.py``).  The K-grouped scales use the group-major memory layout that the
reference's data generator builds
(tests/test_FP8/test_k_grouped_gemm_channel_expert.py:68-98).

``tests/test_oracle_golden.py`` checks ``oracle/`` against the fixture and
``tests/test_gpu_fp8_rowcol.py`` checks the CUDA kernels against it.  A case the reference
cannot run is recorded with its error text instead of an output.
"""

from __future__ import annotations

import argparse
import sys
import traceback
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
sys.path.insert(0, str(HERE.parents[1]))

from fp8_rowcol_cases import E4, E5, K_CASES, M_CASES, input_hashes, k_case_inputs, m_case_inputs  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="directory that holds the reference's `gemm` package")
    ap.add_argument("--out", default=str(HERE / "fp8_rowcol.pt"))
    args = ap.parse_args()
    ref = Path(args.reference)
    sys.path.insert(0, str(ref))
    if not torch.cuda.is_available():
        raise SystemExit("this script runs the reference's Triton kernels and needs a CUDA GPU")

    from make_golden import lift_functions
    from gemm.FP8.k_grouped_gemm_channel_expert import matmul as ref_matmul
    from gemm.FP8.m_grouped_gemm_channel_expert import gmm_fp8_act_per_channel_w_per_expert as ref_gmm

    casts = lift_functions(ref / "gemm/FP8/m_grouped_gemm_channel_expert.py",
                           ["ceil_div", "per_channel_cast_to_fp8", "per_expert_cast_to_fp8"])
    dev = torch.device("cuda", 0)
    fixture = {"m_grouped": {}, "k_grouped": {}, "device": torch.cuda.get_device_name(0),
               "torch": torch.__version__}
    try:
        import triton

        fixture["triton"] = triton.__version__
    except Exception:  # pragma: no cover
        pass

    for name in M_CASES:
        inp = m_case_inputs(name, casts)
        entry = {"inputs_sha256": input_hashes(inp), "dtype_out": str(inp["dtype_out"])}
        try:
            out = ref_gmm(inp["a8"].to(dev), inp["a_scale"].to(dev), inp["b8"].to(dev),
                          inp["b_scale"].reshape(-1).to(dev), inp["sizes"].to(dev), inp["dtype_out"])
            torch.cuda.synchronize()
            entry["out"] = out.cpu()
            print(f"m_grouped {name}: ok {tuple(out.shape)}", flush=True)
        except Exception as exc:  # the reference could not run this case here
            entry["error"] = f"{type(exc).__name__}: {exc}"[:2000]
            print(f"m_grouped {name}: FAILED\n{traceback.format_exc()}", flush=True)
        fixture["m_grouped"][name] = entry

    for name in K_CASES:
        inp = k_case_inputs(name, casts)
        entry = {"inputs_sha256": input_hashes(inp)}
        g, k_tot = inp["tokens"].numel(), int(inp["tokens"].sum())
        try:
            # group-major memory on the device, logical [M, G] / [N, G] views of it
            xs = inp["x_scale"].t().contiguous().to(dev).t()
            ys = inp["y_scale"].t().contiguous().to(dev).t()
            out = ref_matmul(inp["x8"].to(dev), xs, inp["y8"].to(dev), ys, inp["tokens"].to(dev), inp["m"], inp["n"],
                             k_tot, g, inp["dtype_a"], inp["dtype_b"])
            torch.cuda.synchronize()
            entry["out"] = out.cpu()
            print(f"k_grouped {name}: ok {tuple(out.shape)}", flush=True)
        except Exception as exc:
            entry["error"] = f"{type(exc).__name__}: {exc}"[:2000]
            print(f"k_grouped {name}: FAILED\n{traceback.format_exc()}", flush=True)
        fixture["k_grouped"][name] = entry

    # how far the reference's kernels are from this repository's CPU restatement (information only)
    try:
        import oracle as O

        for name, e in fixture["m_grouped"].items():
            if "out" in e:
                inp = m_case_inputs(name, casts)
                ref_o = O.fp8_rowcol_m_grouped_ref(inp["a8"], inp["a_scale"], inp["b8"], inp["b_scale"], inp["sizes"],
                                                   inp["dtype_out"])
                print(f"m_grouped {name}: rdiff(reference kernel, oracle) = "
                      f"{O.rdiff(e['out'].float(), ref_o.float()):.3e}", flush=True)
        for name, e in fixture["k_grouped"].items():
            if "out" in e:
                inp = k_case_inputs(name, casts)
                ref_o = O.fp8_rowcol_k_grouped_ref(inp["x8"], inp["x_scale"], inp["y8"], inp["y_scale"], inp["tokens"],
                                                   inp["m"], inp["n"], inp["tokens"].numel())
                print(f"k_grouped {name}: rdiff(reference kernel, oracle) = "
                      f"{O.rdiff(e['out'].float(), ref_o.float()):.3e}", flush=True)
    except Exception:
        print(traceback.format_exc(), flush=True)

    out_path = Path(args.out)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    torch.save(fixture, out_path)
    print(out_path, out_path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
