"""Write a ``dataset_distributions.json`` of sequence lengths, plus summary statistics.

    python -m lorafusion_b200.cli.gen_sample_distribution --out datasets/dataset_distributions.json \
        --datasets xsum cnn_dailymail wikisum mix --seeds 0 1 --permutations 4 --num-samples 2000

The reference tokenises XSum / CNN-DailyMail / WikiSum with the model's tokenizer, truncates at
4096 tokens and stores, per dataset and seed, several permutations of the resulting length
list (``benchmarks_paper/gen_sample_distribution.py:93-161,300-420``; layout
``{name: {"seed_<s>": {"permutation_<k>": [len, ...]}}}``).  Datasets and tokenizers are not
available offline, so the lengths are drawn from the named lognormal profiles of
``lorafusion_b200.train.data.NAMED_DISTRIBUTIONS``; ``mix`` interleaves all requested
profiles, ``het`` gives every permutation a different profile.  A histogram chart (SVG) is
written next to the JSON with ``--plot``.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np

from ..train.data import NAMED_DISTRIBUTIONS
from ..utils.plotting import MultiLinePlot


def lengths_for(name: str, pool: list, n: int, seed: int, max_len: int) -> np.ndarray:
    if name in NAMED_DISTRIBUTIONS:
        out = NAMED_DISTRIBUTIONS[name].sample(n, seed)
    elif name == "mix":
        parts = [NAMED_DISTRIBUTIONS[p].sample((n + len(pool) - 1) // len(pool), seed + 17 * i)
                 for i, p in enumerate(pool)]
        out = np.stack(parts, axis=1).reshape(-1)[:n]
    else:
        raise KeyError(f"unknown dataset profile {name!r}; known: {sorted(NAMED_DISTRIBUTIONS)} + mix, het")
    return np.minimum(out, max_len)


def generate(datasets, seeds, permutations: int, num_samples: int, max_len: int = 4096) -> dict:
    pool = [d for d in datasets if d in NAMED_DISTRIBUTIONS] or ["xsum", "cnn_dailymail", "wikisum"]
    result: dict = {}
    for name in datasets:
        result[name] = {}
        for seed in seeds:
            perms = {}
            if name == "het":
                for k in range(permutations):
                    perms[f"permutation_{k + 1}"] = lengths_for(pool[k % len(pool)], pool, num_samples,
                                                                seed * 1000 + k, max_len).tolist()
            else:
                base = lengths_for(name, pool, num_samples, seed, max_len)
                rng = np.random.default_rng(seed)
                for k in range(permutations):
                    perms[f"permutation_{k + 1}"] = (base if k == 0 else rng.permutation(base)).tolist()
            result[name][f"seed_{seed}"] = perms
    return result


def summarize(result: dict) -> list:
    rows = []
    for name, seeds in result.items():
        lens = np.asarray(next(iter(next(iter(seeds.values())).values())))
        rows.append({"dataset": name, "samples": int(lens.size), "mean": float(lens.mean()),
                     "median": float(np.median(lens)), "p95": float(np.percentile(lens, 95)),
                     "max": int(lens.max()), "total_tokens": int(lens.sum())})
    return rows


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="datasets/dataset_distributions.json")
    ap.add_argument("--datasets", nargs="+", default=["xsum", "cnn_dailymail", "wikisum", "mix", "het"])
    ap.add_argument("--seeds", nargs="+", type=int, default=[0])
    ap.add_argument("--permutations", type=int, default=4)
    ap.add_argument("--num-samples", type=int, default=2000)
    ap.add_argument("--max-len", type=int, default=4096)
    ap.add_argument("--plot", action="store_true", help="also write <out>.svg with the length histograms")
    args = ap.parse_args(argv)
    result = generate(args.datasets, args.seeds, args.permutations, args.num_samples, args.max_len)
    out = Path(args.out)
    out.parent.mkdir(parents=True, exist_ok=True)
    out.write_text(json.dumps(result))
    for row in summarize(result):
        print(json.dumps(row))
    if args.plot:
        edges = np.linspace(0, args.max_len, 33)
        xs, ys, names = [], [], []
        for name, seeds in result.items():
            lens = np.asarray(next(iter(next(iter(seeds.values())).values())))
            hist, _ = np.histogram(lens, bins=edges)
            names.append(name)
            xs.append(((edges[:-1] + edges[1:]) / 2).tolist())
            ys.append((hist / max(hist.sum(), 1)).tolist())
        MultiLinePlot(names, xs, ys, title="sequence-length distributions", xlabel="tokens",
                      ylabel="fraction of samples").save(out.with_suffix(".svg"))
    return result


if __name__ == "__main__":
    main()
