"""Decoder-layer benchmark: forward+backward time of N layers with 1 or several adapters.

    python -m lorafusion_b200.cli.bench_layer --model llama-3.1-8b --layers 2 --seq-len 512 \
        --batch-sizes 4 8 16 --num-adapters 1 4

Counterpart of ``benchmarks_paper/bench_transformer_layer.py``; rows are appended to a CSV with
the reference's columns ``Mode,Model,BatchSize,SeqLength,NumAdapters,TimeMs,
ThroughputTokensPerSec`` (``bench_transformer_layer.py:296-304``).  ``--profile-only`` runs
the step a few times without timing (for Nsight Compute).
"""

from __future__ import annotations

import argparse
import csv
import json
from pathlib import Path

import torch

from ..models.config import AdapterSpec, get_model_config
from ..models.decoder import DecoderStage
from ..ops import _native
from ..train.data import MicroBatchSpec, build_packed_batch
from ..utils.benchmark import benchmark


def main(argv=None) -> list:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--batch-sizes", nargs="+", type=int, default=[8, 16, 32])
    ap.add_argument("--num-adapters", nargs="+", type=int, default=[1, 4])
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--dropout", type=float, default=0.1)
    ap.add_argument("--quantize", action="store_true")
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--number", type=int, default=10)
    ap.add_argument("--csv", default=None)
    ap.add_argument("--profile-only", action="store_true")
    args = ap.parse_args(argv)

    cfg = get_model_config(args.model).with_layers(args.layers)
    rows = []
    for n_ad in args.num_adapters:
        adapters = [AdapterSpec(f"lora_{i}", r=args.rank, dropout=args.dropout) for i in range(n_ad)]
        stage = DecoderStage(cfg, adapters, "cuda", quantize=args.quantize, recompute=args.recompute,
                             init_b_std=0.01, with_optimizer_state=False)
        for bs in args.batch_sizes:
            per = max(1, bs // n_ad)
            spec = MicroBatchSpec([(a, [args.seq_len] * per) for a in range(n_ad)])
            batch = build_packed_batch(spec, adapters, cfg.vocab_size, "cuda", seed=bs)
            if args.profile_only:
                for _ in range(args.number):
                    stage.forward_backward(batch)
                torch.cuda.synchronize()
                continue
            t = benchmark(lambda: stage.forward_backward(batch), warmup=args.warmup, number=args.number)
            toks = spec.total_tokens
            rows.append({"Mode": "FusedMultiLoRA" if n_ad > 1 else "FusedLoRA", "Model": cfg.name,
                         "BatchSize": per * n_ad, "SeqLength": args.seq_len, "NumAdapters": n_ad,
                         "TimeMs": t * 1e3, "ThroughputTokensPerSec": toks / t})
            print(json.dumps(rows[-1]))
        del stage
        torch.cuda.empty_cache()
    _native.check_device_errors()
    if args.csv and rows:
        p = Path(args.csv)
        p.parent.mkdir(parents=True, exist_ok=True)
        new = not p.exists()
        with open(p, "a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(rows[0]))
            if new:
                w.writeheader()
            w.writerows(rows)
    return rows


if __name__ == "__main__":
    main()
