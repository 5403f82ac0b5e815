"""Collect ``results.csv`` files of training runs into one table, compute speed-ups against a
baseline run and optionally draw the end-to-end and scaling figures.

    python -m lorafusion_b200.cli.parse_results outputs/*/results.csv --baseline-schedule mlora --plot figs/

Counterpart of ``benchmarks_paper/parse_main_results.py`` (reads ``logs/<run>/results.csv``
written by ``scripts/run_single.sh:366-374`` and prints per-model speed-ups) and of
``plots/evaluation-fig-1-end-to-end.py`` / ``evaluation-fig-3-scaling.py``.  A row is one
line of ``results.csv`` as written by ``lorafusion_b200.cli.train``.
"""

from __future__ import annotations

import argparse
import csv
import json
from collections import defaultdict
from pathlib import Path

from ..utils.benchmark import tabulate_2d_benchmark_results
from ..utils.plotting import GroupedBarChart, MultiLinePlot


def load_rows(paths) -> list:
    rows = []
    for p in paths:
        with open(p, newline="") as f:
            for r in csv.DictReader(f):
                r["source"] = str(p)
                for k in ("world", "adapters", "capacity", "microbatches"):
                    r[k] = int(float(r[k]))
                for k in ("tokens", "time_ms", "throughput_tokens_per_s", "throughput_per_gpu", "peak_memory_gib"):
                    r[k] = float(r[k])
                rows.append(r)
    return rows


def best_by_config(rows) -> dict:
    """Highest throughput per (model, world, layout, schedule)."""
    best: dict = {}
    for r in rows:
        key = (r["model"], r["world"], r["layout"], r["schedule"])
        if key not in best or r["throughput_tokens_per_s"] > best[key]["throughput_tokens_per_s"]:
            best[key] = r
    return best


def speedups(best: dict, baseline_schedule: str) -> list:
    out = []
    for (model, world, layout, sched), r in sorted(best.items()):
        if sched == baseline_schedule:
            continue
        base = best.get((model, world, layout, baseline_schedule))
        out.append({"model": model, "world": world, "layout": layout, "schedule": sched,
                    "tokens_per_s": r["throughput_tokens_per_s"],
                    "baseline_tokens_per_s": base["throughput_tokens_per_s"] if base else None,
                    "speedup": r["throughput_tokens_per_s"] / base["throughput_tokens_per_s"] if base else None})
    return out


def main(argv=None) -> list:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("results", nargs="+", help="results.csv files")
    ap.add_argument("--baseline-schedule", default="mlora")
    ap.add_argument("--plot", default=None, help="directory for end_to_end.svg and scaling.svg")
    ap.add_argument("--csv", default=None)
    args = ap.parse_args(argv)
    rows = load_rows(args.results)
    best = best_by_config(rows)
    keys = sorted(best)
    names = [f"{m} x{w} {lay} [{s}]" for m, w, lay, s in keys]
    vals = [[best[k]["throughput_tokens_per_s"], best[k]["throughput_per_gpu"], best[k]["peak_memory_gib"]] for k in keys]
    print(tabulate_2d_benchmark_results(names, ["tokens/s", "tokens/s/GPU", "peak GiB"], vals, fmt="{:.1f}",
                                        csv_path=args.csv, title="best run per configuration"))
    sp = speedups(best, args.baseline_schedule)
    for row in sp:
        print(json.dumps(row))
    if args.plot:
        out = Path(args.plot)
        models = sorted({k[0] for k in keys})
        scheds = sorted({k[3] for k in keys})
        table = [[max((best[k]["throughput_tokens_per_s"] for k in keys if k[0] == m and k[3] == s), default=0.0)
                  for m in models] for s in scheds]
        GroupedBarChart(models, scheds, table, title="end-to-end throughput", ylabel="tokens/s").save(
            out / "end_to_end.svg")
        per_model = defaultdict(dict)
        for (m, w, lay, s), r in best.items():
            per_model[f"{m} [{s}]"][w] = max(per_model[f"{m} [{s}]"].get(w, 0.0), r["throughput_tokens_per_s"])
        series = sorted(per_model)
        MultiLinePlot(series, [sorted(per_model[s]) for s in series],
                      [[per_model[s][w] for w in sorted(per_model[s])] for s in series], logx=True,
                      title="scaling", xlabel="GPUs", ylabel="tokens/s").save(out / "scaling.svg")
    return sp


if __name__ == "__main__":
    main()
