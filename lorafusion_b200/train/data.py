"""Synthetic data: sequence-length distributions, mock datasets and packed microbatches.

The reference trains on random token ids and only takes *length distributions* from real
datasets (``lorafusion/train/training_utils.py:903-1347``, ``lorafusion/utils/hf.py:6-121``,
``benchmarks_paper/gen_sample_distribution.py:93-161``).  With no dataset access the length
distributions here are lognormal (median, sigma, clip range), which is also what the
reference's imbalance simulator uses for its random-data mode
(``benchmarks_paper/imbalance_simulator/main_random_data.py:15-61``).

A packed microbatch groups tokens by adapter; every adapter segment is padded to a multiple
of 128 tokens with a dummy sequence whose labels are ignored, so padding never mixes with
real sequences in attention and contributes zero gradient.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional, Sequence

import numpy as np
import torch

from ..models.config import AdapterSpec
from ..models.decoder import PackedBatch
from ..ops.attention import build_attn_tiles
from ..ops.batch_info import prepare_multi_lora_batch_info

IGNORE_INDEX = -100
TILE = 128


@dataclass(frozen=True)
class LengthDistribution:
    """Lognormal sequence lengths: ``exp(N(ln median, sigma))`` clipped to ``[lo, hi]``."""

    median: float = 512.0
    sigma: float = 0.6
    lo: int = 64
    hi: int = 4096
    name: str = "lognormal"

    def sample(self, n: int, seed: int = 0) -> np.ndarray:
        rng = np.random.default_rng(seed)
        x = rng.lognormal(mean=np.log(self.median), sigma=self.sigma, size=n)
        return np.clip(np.rint(x), self.lo, self.hi).astype(np.int64)


# stand-ins for the reference's dataset names (XSum / CNN-DailyMail / WikiSum token-length
# profiles are approximated by lognormals of increasing median)
NAMED_DISTRIBUTIONS = {
    "xsum": LengthDistribution(512, 0.5, 32, 4096, "xsum"),
    "cnn_dailymail": LengthDistribution(1024, 0.5, 32, 4096, "cnn_dailymail"),
    "wikisum": LengthDistribution(2048, 0.6, 32, 4096, "wikisum"),
    "short": LengthDistribution(256, 0.5, 32, 8192, "short"),
    "medium": LengthDistribution(512, 0.6, 32, 8192, "medium"),
    "long": LengthDistribution(1024, 0.7, 32, 8192, "long"),
    "xlong": LengthDistribution(2048, 0.8, 32, 8192, "xlong"),
}


class MockDataset:
    """A list of sample lengths for one adapter (job), drawn once from a distribution."""

    def __init__(self, lengths: Sequence[int], name: str = "mock"):
        self.lengths = [int(v) for v in lengths]
        self.name = name

    @classmethod
    def from_distribution(cls, dist: LengthDistribution, num_samples: int, seed: int = 0) -> "MockDataset":
        return cls(dist.sample(num_samples, seed).tolist(), dist.name)

    @classmethod
    def from_distribution_file(cls, path: str | Path, name: str, seed: int = 0, permutation: int = 1):
        """Read the reference's ``dataset_distributions.json`` layout:
        ``{name: {"seed_<s>": {"permutation_<k>": [len, ...]}}}``."""
        data = json.loads(Path(path).read_text())
        return cls(data[name][f"seed_{seed}"][f"permutation_{permutation}"], name)

    def __len__(self) -> int:
        return len(self.lengths)

    def global_batches(self, global_batch_size: int) -> list[list[int]]:
        n = len(self.lengths) // global_batch_size
        return [self.lengths[i * global_batch_size:(i + 1) * global_batch_size] for i in range(n)]


@dataclass
class MicroBatchSpec:
    """Host description of a microbatch: ``segments[i] = (adapter_idx, [sequence lengths])``;
    at most one segment per adapter."""

    segments: list = field(default_factory=list)
    is_empty_marker: bool = False
    total_multiple: int = TILE   # the packed length is rounded up to this (128 x tp under TP)

    @property
    def total_tokens(self) -> int:
        return sum(sum(lens) for _, lens in self.segments)

    @property
    def segment_padded_tokens(self) -> int:
        return sum(((sum(lens) + TILE - 1) // TILE) * TILE for _, lens in self.segments)

    @property
    def tail_pad_tokens(self) -> int:
        """Adapter-less filler rows appended so that the total is a multiple of
        ``total_multiple`` (their labels are ignored, they form their own sequence)."""
        return (-self.segment_padded_tokens) % max(self.total_multiple, TILE)

    @property
    def padded_total_tokens(self) -> int:
        return self.segment_padded_tokens + self.tail_pad_tokens


def stage_host_batch(spec: MicroBatchSpec, vocab_size: int, seed: int, pin: bool = True):
    """Create the token-level arrays of a microbatch in (pinned) host memory.

    Returns ``(host [3, T] int32 = ids | labels | positions, cu_seqlens, seg_tokens)``."""
    rng = np.random.default_rng(seed)
    T = spec.padded_total_tokens
    host = torch.empty((3, T), dtype=torch.int32, pin_memory=pin and torch.cuda.is_available())
    arr = host.numpy()
    ids, labels, pos = arr[0], arr[1], arr[2]
    ids[:] = rng.integers(0, vocab_size, size=T, dtype=np.int64)
    labels[:] = IGNORE_INDEX
    cu = [0]
    seg_tokens = []
    t = 0
    for _, lens in spec.segments:
        seg_start = t
        for n in lens:
            pos[t:t + n] = np.arange(n)
            labels[t:t + n - 1] = ids[t + 1:t + n]
            t += n
            cu.append(t)
        real = t - seg_start
        seg_tokens.append(real)
        pad = (-real) % TILE
        if pad:
            pos[t:t + pad] = np.arange(pad)
            t += pad
            cu.append(t)
    tail = spec.tail_pad_tokens
    if tail:
        pos[t:t + tail] = np.arange(tail)
        t += tail
        cu.append(t)
    assert t == T
    return host, cu, seg_tokens


def build_packed_batch(spec: MicroBatchSpec, adapters: Sequence[AdapterSpec], vocab_size: int, device,
                       seed: int = 0, dropout_seed: Optional[int] = None, host=None) -> PackedBatch:
    """Materialise a microbatch on ``device``: one pinned staging buffer, one H2D copy for
    the token arrays and one for the block table."""
    device = torch.device(device)
    if host is None:
        host = stage_host_batch(spec, vocab_size, seed, pin=device.type == "cuda")
    host_arr, cu, seg_tokens = host
    dev = host_arr.to(device, non_blocking=True)
    idx = [a for a, _ in spec.segments]
    if spec.tail_pad_tokens:
        idx = idx + [-1]
        seg_tokens = list(seg_tokens) + [spec.tail_pad_tokens]
    info = prepare_multi_lora_batch_info(
        seg_tokens, idx, [adapters[a].r if a >= 0 else 0 for a in idx],
        [adapters[a].dropout if a >= 0 else 0.0 for a in idx],
        [adapters[a].scaling if a >= 0 else 0.0 for a in idx], device=device,
        seed=seed if dropout_seed is None else dropout_seed, num_adapters=max(len(adapters), 1),
        micro_batch_info=spec)
    labels_np = host_arr[1].numpy()
    return PackedBatch(input_ids=dev[0], labels=dev[1], position_ids=dev[2], cu_seqlens=cu,
                       attn_tiles=build_attn_tiles(cu, device), info=info,
                       num_real_tokens=spec.total_tokens,
                       num_loss_tokens=int((labels_np != IGNORE_INDEX).sum()))


def h2d_bytes(batch: PackedBatch) -> int:
    """Bytes a microbatch moves host-to-device (token arrays + block table + tile lists)."""
    n = 3 * batch.num_tokens * 4
    n += batch.attn_tiles.tiles.numel() * 4
    n += batch.info.tile_adapter.numel() * 4 * 4 + batch.info.adapter_scale.numel() * 12
    return int(n)


def pack_greedy(lengths_by_adapter: dict[int, list[int]], capacity: int) -> list[MicroBatchSpec]:
    """First-fit-decreasing packing of samples into microbatches of at most ``capacity``
    padded tokens; a quick stand-in when no solver schedule is supplied."""
    items = sorted(((n, a) for a, lens in lengths_by_adapter.items() for n in lens), reverse=True)
    bins: list[dict[int, list[int]]] = []
    for n, a in items:
        placed = False
        for b in bins:
            trial = {k: list(v) for k, v in b.items()}
            trial.setdefault(a, []).append(n)
            padded = sum(((sum(v) + TILE - 1) // TILE) * TILE for v in trial.values())
            if padded <= capacity:
                b.setdefault(a, []).append(n)
                placed = True
                break
        if not placed:
            bins.append({a: [n]})
    return [MicroBatchSpec([(a, lens) for a, lens in sorted(b.items())]) for b in bins]


def pack_balanced_dp_step(samples: Sequence[tuple], world: int, per_rank: int, capacity: int, *,
                          time_limit: float = 0.1, slack: float = 0.04) -> tuple[list, list]:
    """Microbatches of one data-parallel step: every rank gets ``per_rank`` nearly full
    microbatches and about the same attention work.

    ``samples`` = ``[(adapter, length)]``, the pool to draw from (it should hold a little more
    than ``world * per_rank * capacity`` tokens).  Two stages:

    1. Samples are dealt to ranks longest first, each to the rank with the smallest
       ``sum(length^2)`` so far -- the causal-attention cost, the only part of a step that is
       not linear in tokens -- among the ranks whose token budget (``per_rank * capacity``
       plus ``slack``) still has room.  What fits nowhere is a leftover.
    2. Each rank's samples are bin-packed into microbatches of at most ``capacity`` padded
       tokens by the solver (fewest bins, then smallest leftover bin:
       ``solver.schedule.solve_micro_milp_lexicographic``; with some thirty samples per rank
       the branch and bound is exact).  The ``per_rank`` fullest bins are used, the samples
       of any further bin are leftovers.

    Returns ``(specs[rank][i], leftovers)``; leftovers go first into the next step's pool.
    Independent random draws per rank, the alternative, make every step as slow as the rank
    that happened to draw the longest sequences."""
    from ..solver.schedule import solve_micro_milp_lexicographic

    budget = int(per_rank * capacity * (1.0 + slack))
    tokens, cost = [0] * world, [0] * world
    sets: list = [[] for _ in range(world)]
    leftovers = []
    for i in sorted(range(len(samples)), key=lambda i: -samples[i][1]):
        n = samples[i][1]
        cands = [r for r in range(world) if tokens[r] + n <= budget]
        if not cands:
            leftovers.append(samples[i])
            continue
        r = min(cands, key=lambda r: (cost[r], tokens[r]))
        sets[r].append(i)
        tokens[r] += n
        cost[r] += n * n
    dealt = []
    for r in range(world):
        keyed = [(i, samples[i][0], samples[i][1]) for i in sets[r]]
        bins, _ = solve_micro_milp_lexicographic(keyed, capacity, TILE, time_limit)
        if len(bins) < per_rank:
            raise ValueError(f"the pool fills only {len(bins)} microbatches on rank {r}, {per_rank} are needed")
        bins.sort(key=lambda b: -sum(samples[i][1] for i in b))
        leftovers += [samples[i] for b in bins[per_rank:] for i in b]
        specs = []
        for b in bins[:per_rank]:
            per: dict = {}
            for i in sorted(b):
                per.setdefault(samples[i][0], []).append(samples[i][1])
            specs.append(MicroBatchSpec(sorted(per.items())))
        dealt.append(specs)
    return dealt, leftovers
