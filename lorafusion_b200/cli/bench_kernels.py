"""Kernel-level benchmark of the fused LoRA linear layer.

    python -m lorafusion_b200.cli.bench_kernels --shapes 4096x4096 8192x8192 --tokens 8192

For every ``K x N`` shape and token count it times, forward and forward+backward:
``Torch Linear`` (cuBLAS, no adapter), ``Torch LoRA`` (unfused: cuBLAS GEMMs + elementwise
ops + torch dropout), ``FusedLoRA`` (one adapter) and ``FusedMultiLoRA-4x`` (four adapters
sharing the microbatch) -- and, with ``--reference-triton``, the reference's own Triton kernels
compiled for this GPU and composed as the reference composes them
(``cli/reference_kernels.py``; checked against fp32 math before they are timed).  Each arm
runs inside an NVTX range of the reference's names (``RawLinear``, ``RawLoRA``, ``FusedLoRA``,
``FusedMultiLoRA``, ``benchmarks_paper/bench_lora_kernels.py:323,398,466,610``) so that an
Nsight capture can be filtered by arm.  Rows are written in the reference's CSV layout
(``Shape, Torch LoRA, Torch Linear, FlashLoRA`` seconds with rows
``"[MxKxNxr] FWD|FWD+BWD"``, ``benchmarks_paper/bench_lora_kernels.py:899-936``) plus the
multi-adapter column.  ``--profile-only fused_fwd`` runs just one variant a few times, which
is what the Nsight Compute commands under ``profiles/`` call.
"""

from __future__ import annotations

import argparse
import json

import torch

from ..ops import lora_kernels as lk
from ..ops.batch_info import prepare_multi_lora_batch_info, single_adapter_batch_info
from ..ops.lora import LoRAStack, lora_linear_backward, lora_linear_forward
from ..utils.benchmark import benchmark, nvtx_range, tabulate_2d_benchmark_results


def _stack(n, N, K, r, device):
    a = torch.zeros(n, 64, K, device=device, dtype=torch.bfloat16)
    b = torch.zeros(n, N, 64, device=device, dtype=torch.bfloat16)
    a[:, :r] = torch.randn(n, r, K, device=device) * 0.02
    b[:, :, :r] = torch.randn(n, N, r, device=device) * 0.02
    return LoRAStack(a, b, torch.zeros(n, 64, K, device=device), torch.zeros(n, N, 64, device=device))


def make_case(M, K, N, r, p, n_adapters, device="cuda"):
    x = torch.randn(M, K, device=device).to(torch.bfloat16)
    w = (torch.randn(N, K, device=device) * 0.02).to(torch.bfloat16)
    dy = torch.randn(M, N, device=device).to(torch.bfloat16)
    stack = _stack(n_adapters, N, K, r, device)
    if n_adapters == 1:
        info = single_adapter_batch_info(M, r, 2.0, p, device=device)
    else:
        per = (M // n_adapters // 128) * 128
        lens = [per] * (n_adapters - 1) + [M - per * (n_adapters - 1)]
        info = prepare_multi_lora_batch_info(lens, list(range(n_adapters)), [r] * n_adapters, [p] * n_adapters,
                                             [2.0] * n_adapters, device=device)
    return x, w, dy, stack, info


def fused_fwd(x, w, dy, stack, info):
    return lora_linear_forward(x, w, stack, info, stream_id=1)


def fused_fwd_bwd(x, w, dy, stack, info):
    y, s = lora_linear_forward(x, w, stack, info, stream_id=1)
    return lora_linear_backward(dy, x, s, w, stack, info, stream_id=1)


def torch_linear(x, w, dy, mode):
    y = x @ w.t()
    if mode == "fwd":
        return y
    return dy @ w


def torch_lora(x, w, dy, a, b, p, mode):
    """Unfused LoRA with cuBLAS GEMMs; the backward is written out (base frozen)."""
    xh = torch.nn.functional.dropout(x, p) if p > 0 else x
    s = xh @ a.t()
    y = x @ w.t()
    y += (s @ b.t()) * 2.0
    if mode == "fwd":
        return y
    ds = (dy @ b) * 2.0
    db = dy.t() @ s * 2.0
    da = ds.t() @ xh
    dx = dy @ w
    dx += (ds @ a) if p == 0 else (ds @ a) * (xh != 0) / (1 - p)
    return dx, da, db


def run_nf4_compare(args):
    """Base GEMM on an NF4 weight: dequantise to scratch then the bf16 kernel, against the
    kernel that expands NF4 inside its main loop, forward and input gradient."""
    from ..ops import nf4
    from ..ops.lora import materialize_weight, set_nf4_fused_max_tokens

    rows = []
    for shape in args.shapes:
        K, N = (int(v) for v in shape.lower().split("x"))
        w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
        qw = nf4.quantize_nf4(w)
        qw.fp32_block_scales()
        for M in args.tokens:
            x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            dy = torch.randn(M, N, device="cuda").to(torch.bfloat16)
            kw = dict(warmup=args.warmup, number=args.number, flush=True)

            def scratch_fwd():
                set_nf4_fused_max_tokens(0)
                return lk.base_lora_fwd(x, materialize_weight(qw, M), None, None, tile_adapter=None)

            def fused_fwd_():
                return lk.base_lora_fwd(x, qw, None, None, tile_adapter=None)

            def scratch_dx():
                set_nf4_fused_max_tokens(0)
                return lk.base_lora_dx(dy, materialize_weight(qw, M), None, None, tile_adapter=None)

            def fused_dx():
                return lk.base_lora_dx(dy, qw, None, None, tile_adapter=None)

            if args.profile_only == "nf4_fwd":
                for _ in range(args.number):
                    fused_fwd_()
                torch.cuda.synchronize()
                return []
            row = {"shape": f"[{M}x{K}x{N}] NF4", "scratch_fwd_s": benchmark(scratch_fwd, **kw),
                   "fused_fwd_s": benchmark(fused_fwd_, **kw), "scratch_dx_s": benchmark(scratch_dx, **kw),
                   "fused_dx_s": benchmark(fused_dx, **kw)}
            row["fused_fwd_tflops"] = 2 * M * K * N / row["fused_fwd_s"] / 1e12
            rows.append(row)
            print(json.dumps(row))
    from ..ops import _native

    _native.check_device_errors()
    return rows


def reference_triton_arms(x, w, dy, a, b, M, K, N, args, mode, kw) -> dict:
    """Times of the reference's kernels for one shape and pass, single adapter and four
    adapters; ``{"ref_triton_error": message}`` when they cannot be imported or compiled."""
    from . import reference_kernels as rk

    try:
        rk.load_reference(args.reference_path)
        alpha, p, r = 2.0, args.dropout, args.rank
        out = {}
        if mode == "fwd":  # numerics once per shape, before any timing
            errs = rk.check_single(x, w, a, b, dy, alpha, p)
            out["ref_triton_max_abs_err"] = errs
            if errs["y"] > 0.05 * max(errs["y_scale"], 1.0) or errs["dx"] > 0.05 * max(errs["dx_scale"], 1.0):
                raise RuntimeError(f"reference kernels disagree with fp32 math: {errs}")
        per = (M // 4 // 128) * 128
        lens = [per] * 3 + [M - 3 * per]
        info = rk.ref_multi_batch_info(lens, [r] * 4, [alpha] * 4, [p] * 4)
        a4 = [(torch.randn(r, K, device=x.device) * 0.02).to(x.dtype) for _ in range(4)]
        b4 = [(torch.randn(N, r, device=x.device) * 0.02).to(x.dtype) for _ in range(4)]

        def single():
            y, saved = rk.ref_lora_forward(x, w, a, b, alpha, p)
            return y if mode == "fwd" else rk.ref_lora_backward(dy, w, a, b, alpha, p, saved)

        def multi():
            y, saved = rk.ref_multi_lora_forward(x, w, a4, b4, info)
            return y if mode == "fwd" else rk.ref_multi_lora_backward(dy, w, a4, b4, info, saved)

        with nvtx_range("RefTritonLoRA"):
            out["ref_triton_lora_s"] = benchmark(single, **kw)
        with nvtx_range("RefTritonMultiLoRA"):
            out["ref_triton_multi_lora_4x_s"] = benchmark(multi, **kw)
        return out
    except Exception as e:  # noqa: BLE001 - foreign code: report, keep the other arms
        return {"ref_triton_error": f"{type(e).__name__}: {str(e)[:400]}"}


def run(args):
    if args.nf4_compare or args.profile_only == "nf4_fwd":
        return run_nf4_compare(args)
    torch.manual_seed(0)
    results = []
    for shape in args.shapes:
        K, N = (int(v) for v in shape.lower().split("x"))
        for M in args.tokens:
            x, w, dy, stack1, info1 = make_case(M, K, N, args.rank, args.dropout, 1)
            _, _, _, stack4, info4 = make_case(M, K, N, args.rank, args.dropout, 4)
            a, b = stack1.a[0, :args.rank].contiguous(), stack1.b[0, :, :args.rank].contiguous()
            for mode in ("fwd", "fwd_bwd"):
                if args.profile_only:
                    fn = {"fused_fwd": lambda: fused_fwd(x, w, dy, stack1, info1),
                          "fused_fwd_bwd": lambda: fused_fwd_bwd(x, w, dy, stack1, info1),
                          "multi_fwd_bwd": lambda: fused_fwd_bwd(x, w, dy, stack4, info4)}[args.profile_only]
                    for _ in range(args.number):
                        fn()
                    torch.cuda.synchronize()
                    return []
                kw = dict(warmup=args.warmup, number=args.number, flush=True)
                with nvtx_range("RawLinear"):
                    t_lin = benchmark(lambda: torch_linear(x, w, dy, mode), **kw)
                with nvtx_range("RawLoRA"):
                    t_tl = benchmark(lambda: torch_lora(x, w, dy, a, b, args.dropout, mode), **kw)
                f1 = fused_fwd if mode == "fwd" else fused_fwd_bwd
                with nvtx_range("FusedLoRA"):
                    t_f1 = benchmark(lambda: f1(x, w, dy, stack1, info1), **kw)
                with nvtx_range("FusedMultiLoRA"):
                    t_f4 = benchmark(lambda: f1(x, w, dy, stack4, info4), **kw)
                flops = (2 if mode == "fwd" else 4) * M * K * N
                row = {"shape": f"[{M}x{K}x{N}x{args.rank}] {'FWD' if mode == 'fwd' else 'FWD+BWD'}",
                       "torch_lora_s": t_tl, "torch_linear_s": t_lin, "fused_lora_s": t_f1,
                       "fused_multi_lora_4x_s": t_f4, "speedup_vs_torch_lora": t_tl / t_f1,
                       "fused_tflops": flops / t_f1 / 1e12, "linear_tflops": flops / t_lin / 1e12}
                if args.reference_triton:
                    row.update(reference_triton_arms(x, w, dy, a, b, M, K, N, args, mode, kw))
                    if "ref_triton_lora_s" in row:
                        row["speedup_vs_ref_triton"] = row["ref_triton_lora_s"] / t_f1
                        row["multi_speedup_vs_ref_triton"] = row["ref_triton_multi_lora_4x_s"] / t_f4
                results.append(row)
    rows = [r["shape"] for r in results]
    cols = ["Torch LoRA", "Torch Linear", "FlashLoRA", "MultiLoRA-4x"]
    vals = [[r["torch_lora_s"], r["torch_linear_s"], r["fused_lora_s"], r["fused_multi_lora_4x_s"]] for r in results]
    if args.reference_triton and all("ref_triton_lora_s" in r for r in results):
        cols += ["Ref-Triton LoRA", "Ref-Triton MultiLoRA-4x"]
        vals = [v + [r["ref_triton_lora_s"], r["ref_triton_multi_lora_4x_s"]] for v, r in zip(vals, results)]
    print(tabulate_2d_benchmark_results(rows, cols, vals, fmt="{:.6f}", csv_path=args.csv, title="seconds"))
    for r in results:
        print(json.dumps(r))
    from ..ops import _native

    _native.check_device_errors()
    return results


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shapes", nargs="+", default=["4096x4096", "5120x5120", "8192x8192"], help="KxN")
    ap.add_argument("--tokens", nargs="+", type=int, default=[8192])
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--dropout", type=float, default=0.1)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--number", type=int, default=20)
    ap.add_argument("--csv", default=None)
    ap.add_argument("--nf4-compare", action="store_true",
                    help="time the NF4 base GEMM: dequantise-to-scratch + bf16 kernel vs NF4 expanded in the main loop")
    ap.add_argument("--reference-triton", action="store_true",
                    help="also time the reference's own Triton kernels on this GPU (needs a copy of its package)")
    ap.add_argument("--reference-path", default=None, help="directory that holds the reference's lorafusion package")
    ap.add_argument("--profile-only", default=None,
                    choices=["fused_fwd", "fused_fwd_bwd", "multi_fwd_bwd", "nf4_fwd"])
    run(ap.parse_args(argv))


if __name__ == "__main__":
    main()
