"""Per-figure drivers: the five evaluation figures of the reference, drawn as SVG from the files
this framework's benchmarks write.

    python -m lorafusion_b200.cli.figures end-to-end  --results outputs/parsed_main.json --out figs/
    python -m lorafusion_b200.cli.figures scaling     --results SCALE.json --out figs/
    python -m lorafusion_b200.cli.figures kernel-perf --results outputs/kernel_perf/kernels.jsonl --out figs/
    python -m lorafusion_b200.cli.figures layer-perf  --results outputs/layer_perf/layers.jsonl --out figs/
    python -m lorafusion_b200.cli.figures kernel-dram --results outputs/kernel_perf/ncu_dram.json --out figs/

Counterparts of ``benchmarks_paper/plots/evaluation-fig-1-end-to-end.py`` (grouped bars per
model and dataset, four methods), ``evaluation-fig-3-scaling.py`` (throughput at 4 / 8 / 16
GPUs per method), ``evaluation-fig-5-kernel-perf.py`` (kernel time against tokens, one line per
arm), ``evaluation-fig-6-layer-perf.py`` (decoder-layer time against tokens) and
``evaluation-fig-7-kernel-ncu-profile.py`` (DRAM traffic per arm and shape).  Like those
scripts, every driver falls back to the reference's published numbers (``--demo``) so that a
figure can be drawn before anything has been measured; the published numbers are the ones the
reference hard-codes in those files.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

from ..utils.plotting import GroupedBarChart, MultiLinePlot

METHODS = ["Megatron-LM-FSDP", "Megatron-LM-PP", "mLoRA", "LoRAFusion"]
DATASETS = ["XSUM", "CNNDM", "WikiSum", "Mixed", "Het"]

# published by the reference (plots/evaluation-fig-1-end-to-end.py:47-67), tokens/s
PUBLISHED_END_TO_END = {
    "Llama-3.1-8B (1 x H100)": [[12353.35, None, None, 14874.99], [12231.68, None, None, 14595.14],
                                [9754.33, None, None, 13920.32], [10743.86, None, None, 14403.5],
                                [11270.81, None, None, 14157.83]],
    "Qwen-2.5-32B (2 x H100)": [[3021.52, 2882.46, 4232.88, 4968.81], [3640.74, 3246.74, 4347.63, 4972.94],
                                [3941.92, 3389.00, 4083.53, 4946.70], [3543.74, 3122.09, 4099.92, 5120.85],
                                [3536.98, 3160.07, 4020.31, 4955.23]],
    "Llama-3.1-70B (4 x H100)": [[2696.72, 2336.50, 3901.68, 4892.90], [3475.51, 2567.77, 3989.42, 5182.99],
                                 [3124.19, 2985.42, 3868.17, 5073.56], [3142.48, 2491.07, 3746.07, 5115.41],
                                 [3109.73, 2595.19, 3517.25, 5136.16]],
}
# plots/evaluation-fig-3-scaling.py:58-60, 70B mixed, DP scaling, tokens/s
PUBLISHED_SCALING = {4: [3142.48, 2491.07, 3746.07, 5115.41], 8: [5718.00, 4295.79, 6230.87, 9936.74],
                     16: [10381.60, 8160.81, 13511.95, 18906.69]}
# plots/evaluation-fig-7-kernel-ncu-profile.py:49-51, GiB moved forward + backward
PUBLISHED_DRAM = {"8192x4096x4096": [2.008, 1.258, 1.262], "8192x5120x5120": [2.771, 1.836, 1.838],
                  "8192x8192x8192": [5.289, 4.044, 4.054]}


def _read_jsonl(path) -> list:
    rows = []
    for line in Path(path).read_text().splitlines():
        line = line.strip()
        if line.startswith("{"):
            try:
                rows.append(json.loads(line))
            except ValueError:
                pass
    return rows


def fig_end_to_end(args) -> list:
    """``--results``: JSON ``{model title: [[per-method tokens/s] per dataset]}`` (method order as
    ``METHODS``, ``null`` = not run), e.g. assembled from ``cli.parse_results`` output."""
    data = PUBLISHED_END_TO_END if args.demo or not args.results else json.loads(Path(args.results).read_text())
    out = []
    for title, table in data.items():
        methods = [m for j, m in enumerate(METHODS) if any(row[j] is not None for row in table)]
        cols = [j for j, m in enumerate(METHODS) if m in methods]
        values = [[(row[j] or 0.0) for row in table] for j in cols]
        chart = GroupedBarChart(DATASETS[:len(table)], methods, values, title=title, ylabel="tokens/s")
        out.append(chart.save(Path(args.out) / f"fig1_end_to_end_{title.split()[0].lower()}.svg"))
    return out


def fig_scaling(args) -> list:
    """``--results``: either ``{gpus: [per-method tokens/s]}`` or a scaling record with
    ``scaling.values`` = ``{gpus: tokens/s}`` of this framework (drawn against the published
    LoRAFusion line scaled per GPU)."""
    if args.demo or not args.results:
        gpus = sorted(PUBLISHED_SCALING)
        series, ys = METHODS, [[PUBLISHED_SCALING[g][j] for g in gpus] for j in range(4)]
        xs = [gpus] * 4
    else:
        data = json.loads(Path(args.results).read_text())
        vals = data.get("scaling", {}).get("values") or data
        vals = {int(k): v for k, v in vals.items()}
        gpus = sorted(vals)
        if isinstance(vals[gpus[0]], list):
            series, ys, xs = METHODS, [[vals[g][j] for g in gpus] for j in range(4)], [gpus] * 4
        else:
            per_gpu_ref = PUBLISHED_SCALING[8][3] / 8
            series = ["this framework (B200)", "ideal from 1 GPU", "reference LoRAFusion (H100, published per GPU)"]
            ys = [[vals[g] for g in gpus], [vals[gpus[0]] / gpus[0] * g for g in gpus], [per_gpu_ref * g for g in gpus]]
            xs = [gpus] * 3
    chart = MultiLinePlot(series, xs, ys, logx=True, title="Llama-3.1-70B, four adapters: scaling", xlabel="GPUs",
                          ylabel="tokens/s")
    return [chart.save(Path(args.out) / "fig3_scaling.svg")]


def fig_kernel_perf(args) -> list:
    """``--results``: the JSON lines ``cli.bench_kernels`` prints (one per shape and pass)."""
    if args.demo or not args.results:
        raise SystemExit("kernel-perf has no published table (the reference reads CSVs produced at run time); "
                         "pass --results")
    rows = _read_jsonl(args.results)
    arms = [("torch_linear_s", "Torch Linear"), ("torch_lora_s", "Torch LoRA"), ("ref_triton_lora_s", "Reference Triton"),
            ("fused_lora_s", "FusedLoRA"), ("fused_multi_lora_4x_s", "FusedMultiLoRA-4x")]
    out = []
    groups: dict = {}
    for r in rows:
        dims, mode = r["shape"].split("] ")
        m, k, n, _ = (int(v) for v in dims.strip("[").split("x"))
        groups.setdefault((k, n, mode), []).append((m, r))
    for (k, n, mode), pts in sorted(groups.items()):
        pts.sort(key=lambda t: t[0])
        have = [(key, name) for key, name in arms if all(key in r for _, r in pts)]
        chart = MultiLinePlot([name for _, name in have], [[m for m, _ in pts]] * len(have),
                              [[r[key] * 1e3 for _, r in pts] for key, _ in have],
                              title=f"LoRA linear {k} x {n}, {mode}", xlabel="tokens", ylabel="ms")
        out.append(chart.save(Path(args.out) / f"fig5_kernel_perf_{k}x{n}_{mode.replace('+', '_').lower()}.svg"))
    return out


def fig_layer_perf(args) -> list:
    """``--results``: the JSON lines ``cli.bench_layer`` prints (``model``, ``tokens``,
    ``fwd_bwd_ms`` ...); drawn per model against the reference's profiled H100 layer times
    (``lorafusion/simulator/configs/*.yaml:17-29``) when tokens match."""
    if args.demo or not args.results:
        raise SystemExit("layer-perf needs --results (the reference reads CSVs produced at run time)")
    rows = []
    for r in _read_jsonl(args.results):
        if "Model" in r:   # rows of cli.bench_layer: a whole truncated model, not one layer
            r = {"model": r["Model"], "tokens": r["BatchSize"] * r["SeqLength"], "ms": r["TimeMs"],
                 "what": f"{r.get('Mode', '')} run".strip()}
        rows.append(r)
    ref = {"llama-3.1-8b": {4096: 9.08, 8192: 17.39}, "qwen2.5-32b": {4096: 17.22, 8192: 34.07},
           "llama-3.1-70b": {4096: 27.36, 8192: 54.08}}
    out = []
    for model in sorted({r["model"] for r in rows}):
        pts = sorted(((r["tokens"], r) for r in rows if r["model"] == model), key=lambda t: t[0])
        key = next((k for k in ("layer_fwd_bwd_ms", "fwd_bwd_ms", "ms") if k in pts[0][1]), None)
        if key is None:
            continue
        series, xs, ys = ["this framework (B200)"], [[t for t, _ in pts]], [[r[key] for _, r in pts]]
        if model in ref and key == "layer_fwd_bwd_ms":
            series.append("reference (H100, profiled)")
            xs.append(sorted(ref[model]))
            ys.append([ref[model][t] for t in sorted(ref[model])])
        chart = MultiLinePlot(series, xs, ys, title=f"{model}: forward + backward", xlabel="tokens", ylabel="ms")
        out.append(chart.save(Path(args.out) / f"fig6_layer_perf_{model}.svg"))
    return out


def fig_kernel_dram(args) -> list:
    """``--results``: JSON ``{"MxKxN": [Torch LoRA, FusedLoRA, FusedMultiLoRA] GiB}`` as summarised
    from Nsight Compute ``dram__bytes_read.sum + dram__bytes_write.sum`` (``cli.summarize_ncu``)."""
    data = PUBLISHED_DRAM if args.demo or not args.results else json.loads(Path(args.results).read_text())
    shapes = list(data)
    arms = ["Torch LoRA", "FusedLoRA", "FusedMultiLoRA"]
    chart = GroupedBarChart(shapes, arms, [[data[s][j] for s in shapes] for j in range(3)],
                            title="DRAM traffic, forward + backward", ylabel="GiB")
    return [chart.save(Path(args.out) / "fig7_kernel_dram.svg")]


FIGURES = {"end-to-end": fig_end_to_end, "scaling": fig_scaling, "kernel-perf": fig_kernel_perf,
           "layer-perf": fig_layer_perf, "kernel-dram": fig_kernel_dram}


def main(argv=None) -> list:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("figure", choices=sorted(FIGURES))
    ap.add_argument("--results", default=None)
    ap.add_argument("--out", default="figs")
    ap.add_argument("--demo", action="store_true", help="draw the reference's published numbers")
    args = ap.parse_args(argv)
    Path(args.out).mkdir(parents=True, exist_ok=True)
    paths = FIGURES[args.figure](args)
    for p in paths:
        print(p)
    return paths


if __name__ == "__main__":
    main()
