"""Kernel tuner: times the fused GEMM variants over their launch parameters and writes the
best choice per shape to a JSON file.

    python -m lorafusion_b200.cli.tune --shapes 8192x8192 8192x28672 --tokens 16384 --out results/tuning_results.json

The winners are also merged into the launch-parameter table of this GPU
(``ops/tile_config.py``, file ``lorafusion_b200/ops/tuned/<gpu name>.json`` unless ``--table``
says otherwise), which the launchers read from then on.

Counterpart of ``tools/tune_kernels.py`` (which sweeps Triton tile sizes / stages / warps,
``tune_kernels.py:96-133``).  The tcgen05 kernels have fixed 128-row tiles; what is swept
here is the N tile (128 / 256), the L2 grouping of M tiles (``group_m``), the number of
persistent CTAs, and for the dropout dX kernel the accumulator layout (two double-buffered
128-column accumulators or two single-buffered 256-column ones).
"""

from __future__ import annotations

import argparse
import itertools
import json
from pathlib import Path

import torch

from ..ops import _native as nv
from ..ops.gemm import launch_gemm
from ..utils.benchmark import benchmark


def tune_shape(M: int, K: int, N: int, warmup: int, number: int) -> dict:
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    dy = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    s = (torch.randn(M, 64, device="cuda") * 0.1).to(torch.bfloat16)
    b2 = (torch.randn(N, 64, device="cuda") * 0.02).to(torch.bfloat16)
    a2 = (torch.randn(64, K, device="cuda") * 0.02).to(torch.bfloat16)
    y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * M * K * N
    out = {"shape": f"{M}x{K}x{N}", "fwd": [], "dx": [], "dx_dropout": []}
    for bn, gm, ctas in itertools.product((256, 128), (4, 8, 16, 32), (0, 132)):
        t = benchmark(lambda: launch_gemm(a=x, b=w, out=y, M=M, N=N, K=K, a2=s, b2=b2, K2=64, bn=bn, group_m=gm,
                                          max_ctas=ctas), warmup=warmup, number=number)
        out["fwd"].append({"bn": bn, "group_m": gm, "max_ctas": ctas, "ms": t * 1e3, "tflops": flops / t / 1e12})
        t = benchmark(lambda: launch_gemm(a=dy, b=w, out=dx, M=M, N=K, K=N, b_mn=True, b2_mn=True, a2=s, b2=a2,
                                          K2=64, bn=bn, group_m=gm, max_ctas=ctas), warmup=warmup, number=number)
        out["dx"].append({"bn": bn, "group_m": gm, "max_ctas": ctas, "ms": t * 1e3, "tflops": flops / t / 1e12})
    for bn, gm in itertools.product((256, 128), (8, 16)):
        t = benchmark(lambda: launch_gemm(a=dy, b=w, out=dx, M=M, N=K, K=N, b_mn=True, b2_mn=True, a2=s, b2=a2,
                                          K2=64, bn=bn, nacc=2, epi=nv.EPI_BF16_DROPMIX, group_m=gm,
                                          thresh16=6554, inv_keep=1 / 0.9, seed=1, stream_id=1),
                      warmup=warmup, number=number)
        out["dx_dropout"].append({"bn": bn, "group_m": gm, "ms": t * 1e3, "tflops": flops / t / 1e12})
    for k in ("fwd", "dx", "dx_dropout"):
        out[f"best_{k}"] = max(out[k], key=lambda r: r["tflops"])
    return out


def main(argv=None) -> list:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shapes", nargs="+", default=["4096x4096"], help="KxN")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--number", type=int, default=10)
    ap.add_argument("--out", default="results/tuning_results.json")
    ap.add_argument("--table", default=None, help="launch-parameter table to merge the winners into "
                    "(default: the table of this GPU inside the package); 'none' = do not write")
    args = ap.parse_args(argv)
    results = []
    for shape in args.shapes:
        K, N = (int(v) for v in shape.lower().split("x"))
        r = tune_shape(args.tokens, K, N, args.warmup, args.number)
        results.append(r)
        print(json.dumps({k: r[k] for k in ("shape", "best_fwd", "best_dx", "best_dx_dropout")}))
    nv.check_device_errors()
    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    Path(args.out).write_text(json.dumps(results, indent=1))
    if args.table != "none":
        from ..ops import tile_config as tc

        entries = {}
        for r in results:
            M, K, N = (int(v) for v in r["shape"].split("x"))
            # the single-CTA sweep varies bn; the launchers choose bn themselves (256-wide tiles go
            # to the CTA-pair kernel), so only the scheduling parameters of the best 256 row are kept
            for kernel, (m, k, n) in (("fwd", (M, K, N)), ("dx", (M, N, K)), ("dx_dropout", (M, N, K))):
                rows = [x for x in r[kernel] if x["bn"] == 256] or r[kernel]
                best = max(rows, key=lambda x: x["tflops"])
                entries[tc.entry_key(kernel, m, k, n)] = {"group_m": best["group_m"],
                                                          "max_ctas": best.get("max_ctas", 0),
                                                          "tflops": round(best["tflops"], 1)}
        print(f"launch-parameter table: {tc.write_table(entries, None if args.table is None else args.table)}")
    return results


if __name__ == "__main__":
    main()
