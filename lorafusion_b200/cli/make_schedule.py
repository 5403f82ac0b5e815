"""Offline schedule generation (CPU only).

    python -m lorafusion_b200.cli.make_schedule --capacity 16384 --num_adapters 4 \
        --num_pipeline_stages 4 --adapter_to_dataset short medium long xlong \
        --adapter_to_global_batch_size 8 8 8 8 --num_global_batches 16 --out schedules/

Counterpart of ``benchmarks_paper/imbalance_simulator/main_with_datasets.py:144-385``: loads
(or synthesises) per-adapter length lists, groups adapters, packs every (global batch, group)
with the native solver, runs the merge pass, verifies the schedule (inserting no-op
microbatches where the bubble lemma demands), writes ``<name>.json`` + ``<name>.pkl`` and
prints the simulated comparison against the naive / sorted / mLoRA schedules.
"""

from __future__ import annotations

import argparse
import json
import time
from pathlib import Path

from ..simulator import pipeline_sim as ps
from ..solver import schedule as S
from ..train.data import NAMED_DISTRIBUTIONS, MockDataset


def build_data(args) -> list:
    data = []
    for a in range(args.num_adapters):
        name = args.adapter_to_dataset[a % len(args.adapter_to_dataset)]
        gbs = args.adapter_to_global_batch_size[a % len(args.adapter_to_global_batch_size)]
        if args.dataset_path:
            ds = MockDataset.from_distribution_file(args.dataset_path, name, args.seed, args.permutation)
        else:
            ds = MockDataset.from_distribution(NAMED_DISTRIBUTIONS[name], gbs * args.num_global_batches, args.seed + a)
        lens = [min(n, args.capacity) for n in ds.lengths]
        data.append([lens[i * gbs:(i + 1) * gbs] for i in range(min(args.num_global_batches, len(lens) // gbs))])
    return data


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--capacity", type=int, default=16384)
    ap.add_argument("--num_adapters", type=int, default=4)
    ap.add_argument("--num_pipeline_stages", type=int, default=4)
    ap.add_argument("--adapter_to_dataset", nargs="+", default=["short", "medium", "long", "xlong"])
    ap.add_argument("--adapter_to_global_batch_size", nargs="+", type=int, default=[8])
    ap.add_argument("--num_global_batches", type=int, default=8)
    ap.add_argument("--dataset_path", default=None, help="dataset_distributions.json in the reference layout")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--permutation", type=int, default=1)
    ap.add_argument("--time_limit", type=float, default=3.0)
    ap.add_argument("--num_workers", type=int, default=8)
    ap.add_argument("--no_exact", action="store_true", help="greedy first-fit-decreasing only")
    ap.add_argument("--no_merge", action="store_true")
    ap.add_argument("--out", default="schedules")
    ap.add_argument("--name", default=None)
    ap.add_argument("--compare", action="store_true", help="simulate naive / sorted / mLoRA schedules too")
    ap.add_argument("--gantt", default=None, help="write an SVG Gantt chart of the simulated 1F1B run of the schedule")
    args = ap.parse_args(argv)

    data = build_data(args)
    t0 = time.time()
    groups = S.group_adapters(data, args.capacity, num_stages=args.num_pipeline_stages)
    sched = S.packing_data_to_microbatches_micro_milp(
        data, groups, args.capacity, args.num_pipeline_stages, time_limit=args.time_limit,
        use_exact=not args.no_exact, num_workers=args.num_workers)
    if not args.no_merge:
        sched = S.apply_merge_pass_for_adapter_group_step_infos(sched, args.num_pipeline_stages)
    ok, msgs, fixed = S.verify_correctness_of_schedule(data, sched, args.num_pipeline_stages, add_bubble=True)
    if not ok:
        raise SystemExit("invalid schedule: " + "; ".join(msgs))
    ok2, msgs2 = S.verify_correctness_of_schedule(data, fixed, args.num_pipeline_stages)
    if not ok2:
        raise SystemExit("schedule still invalid after no-op insertion: " + "; ".join(msgs2))
    name = args.name or S.schedule_name("-".join(args.adapter_to_dataset), args.capacity, args.num_adapters,
                                        args.num_pipeline_stages, args.adapter_to_global_batch_size[0])
    S.save_schedule(fixed, Path(args.out) / name)
    report = {"name": name, "groups": groups, "solve_seconds": time.time() - t0, **S.schedule_statistics(fixed)}
    if args.compare:
        report["simulation"] = ps.compare_schedules(data, args.capacity, args.num_pipeline_stages,
                                                    time_limit=min(args.time_limit, 0.5))
    if args.gantt:
        from ..utils.plotting import PipelineGantt

        tokens = [0 if m.is_empty_marker else m.padded_total_tokens for m in S.flatten_schedule(fixed)]
        tl = ps.evaluate_schedule_pipeline_parallelism(tokens, args.num_pipeline_stages)
        n_st = args.num_pipeline_stages
        fwd = [[(float(tl.f_start[m, s]), float(tl.f_end[m, s])) for m in range(len(tokens))] for s in range(n_st)]
        bwd = [[(float(tl.b_start[m, s]), float(tl.b_end[m, s])) for m in range(len(tokens))] for s in range(n_st)]
        PipelineGantt(fwd, bwd, title=f"{name}: bubble ratio {tl.bubble_ratio:.3f}", width=1200).save(args.gantt)
        report["gantt"] = str(args.gantt)
        report["simulated_bubble_ratio"] = float(tl.bubble_ratio)
    print(json.dumps(report, indent=2))
    return report


if __name__ == "__main__":
    main()
