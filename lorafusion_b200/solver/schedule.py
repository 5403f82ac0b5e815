"""Multi-adapter microbatch scheduling (CPU side).

Given ``data[adapter][global_batch][sample] = token_length`` the solver produces the ordered
list of microbatches the pipeline executes:

1. ``group_adapters``  pairs adapters with short and long samples ("head-tail") so that the
   groups alternate and leave each adapter enough foreign microbatches between two of its
   global batches (the *bubble lemma*).
2. per (global batch, group) the samples are bin-packed into microbatches under a token
   capacity where every adapter's tokens inside a microbatch are padded to the kernels'
   128-token tile: greedy first-fit-decreasing and an exact two-phase branch and bound
   (fewest bins, then emptiest smallest bin) from the C++ core, keeping the better.
3. a merge pass moves the small leftover microbatch of one group into microbatches of the
   following groups when capacity and the bubble lemma allow.
4. ``verify_correctness_of_schedule`` checks capacity, exact cover, one global batch per
   adapter per microbatch and the bubble lemma, optionally inserting empty no-op
   microbatches where the lemma would be violated.

Same data model and function names as the reference
(``lorafusion/solver/proposed_solver.py:50-396, 617-635, 760-1056, 1363-1575``), with the
CBC MILPs replaced by the native search in ``csrc/solver/packer.cpp``.
"""

from __future__ import annotations

import ctypes as C
import json
import math
import pickle
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from pathlib import Path
from typing import Iterable, Optional, Sequence

import numpy as np

ADAPTER_PADDING_MULTIPLE = 128

SampleKey = tuple  # (adapter_idx, global_batch_idx, sample_idx)


def _pad(n: int, m: int) -> int:
    return 0 if n == 0 else ((n + m - 1) // m) * m


@dataclass
class MicroBatchInfo:
    """One microbatch: ``data_samples[(adapter, global_batch, sample)] = tokens``."""

    data_samples: dict
    max_microbatch_size: int
    adapter_padding_multiple: int = ADAPTER_PADDING_MULTIPLE
    micro_batch_idx: Optional[int] = None
    is_empty_marker: bool = False

    # ---- derived views ------------------------------------------------------------
    @property
    def adapter_group_info(self) -> set:
        return {a for a, _, _ in self.data_samples}

    @property
    def adapter_global_batch_idx_pairs(self) -> set:
        return {(a, g) for a, g, _ in self.data_samples}

    @property
    def adapter_token_lengths_pairs(self) -> dict:
        out: dict = {}
        for (a, _, _), n in self.data_samples.items():
            out.setdefault(a, []).append(n)
        return out

    @property
    def adapter_num_samples_pairs(self) -> dict:
        return {a: len(v) for a, v in self.adapter_token_lengths_pairs.items()}

    @property
    def adapter_num_tokens_pairs(self) -> dict:
        return {a: sum(v) for a, v in self.adapter_token_lengths_pairs.items()}

    @property
    def total_tokens(self) -> int:
        return sum(self.data_samples.values())

    @property
    def padded_adapter_num_tokens_pairs(self) -> dict:
        return {a: _pad(n, self.adapter_padding_multiple) for a, n in self.adapter_num_tokens_pairs.items()}

    @property
    def padded_total_tokens(self) -> int:
        return sum(self.padded_adapter_num_tokens_pairs.values())

    # ---- merging ------------------------------------------------------------------
    def _compatible(self, other: "MicroBatchInfo") -> bool:
        mine = dict(self.adapter_global_batch_idx_pairs)
        for a, g in other.adapter_global_batch_idx_pairs:
            if a in mine and mine[a] != g:
                return False  # two global batches of one adapter cannot share a microbatch
        return True

    def can_full_merge(self, other: "MicroBatchInfo") -> bool:
        if not self._compatible(other):
            return False
        merged = dict(self.data_samples)
        merged.update(other.data_samples)
        return MicroBatchInfo(merged, self.max_microbatch_size, self.adapter_padding_multiple
                              ).padded_total_tokens <= self.max_microbatch_size

    def full_merge(self, other: "MicroBatchInfo") -> bool:
        """Absorb all samples of ``other`` if they fit; ``other`` becomes empty."""
        if not self.can_full_merge(other):
            return False
        self.data_samples.update(other.data_samples)
        other.data_samples = {}
        return True

    def partial_merge(self, other: "MicroBatchInfo") -> int:
        """Move samples of ``other`` (smallest first) into this microbatch while the padded
        size stays within capacity.  Returns the number of samples moved."""
        if not self._compatible(other):
            return 0
        moved = 0
        for key, n in sorted(other.data_samples.items(), key=lambda kv: kv[1]):
            trial = dict(self.data_samples)
            trial[key] = n
            if MicroBatchInfo(trial, self.max_microbatch_size, self.adapter_padding_multiple
                              ).padded_total_tokens > self.max_microbatch_size:
                break
            self.data_samples[key] = n
            del other.data_samples[key]
            moved += 1
        return moved

    # ---- conversions --------------------------------------------------------------
    def segments(self) -> list:
        """``[(adapter, [sample lengths])]`` ordered by adapter: the packed token layout."""
        per: dict = {}
        for (a, _, k), n in sorted(self.data_samples.items()):
            per.setdefault(a, []).append(n)
        return sorted(per.items())

    def to_dict(self) -> dict:
        return {
            "data_samples": [[a, g, k, n] for (a, g, k), n in sorted(self.data_samples.items())],
            "max_microbatch_size": self.max_microbatch_size,
            "adapter_padding_multiple": self.adapter_padding_multiple,
            "micro_batch_idx": self.micro_batch_idx,
            "is_empty_marker": self.is_empty_marker,
            "total_tokens": self.total_tokens,
            "padded_total_tokens": self.padded_total_tokens,
        }

    @classmethod
    def from_dict(cls, d: dict) -> "MicroBatchInfo":
        return cls({(a, g, k): n for a, g, k, n in d["data_samples"]}, d["max_microbatch_size"],
                   d.get("adapter_padding_multiple", ADAPTER_PADDING_MULTIPLE), d.get("micro_batch_idx"),
                   d.get("is_empty_marker", False))

    @classmethod
    def empty_marker(cls, capacity: int) -> "MicroBatchInfo":
        return cls({}, capacity, ADAPTER_PADDING_MULTIPLE, None, True)


@dataclass
class AdapterGroupStepInfo:
    """The microbatches of one adapter group for one global batch, largest first."""

    micro_batch_infos: list = field(default_factory=list)

    def __post_init__(self):
        self.self_update()

    def self_update(self) -> None:
        self.micro_batch_infos = [m for m in self.micro_batch_infos if m.data_samples or m.is_empty_marker]
        self.micro_batch_infos.sort(key=lambda m: m.padded_total_tokens, reverse=True)

    @property
    def adapter_group_info(self) -> set:
        out: set = set()
        for m in self.micro_batch_infos:
            out |= m.adapter_group_info
        return out

    @property
    def internal_adapter_start_end_indices(self) -> dict:
        out = {}
        for a in self.adapter_group_info:
            idx = [i for i, m in enumerate(self.micro_batch_infos) if a in m.adapter_group_info]
            out[a] = (idx[0], idx[-1])
        return out

    @classmethod
    def from_micro_batch_infos_list(cls, infos: list) -> "AdapterGroupStepInfo":
        return cls(list(infos))

    def to_dict(self) -> dict:
        return {"adapter_group_info": sorted(self.adapter_group_info),
                "micro_batch_infos": [m.to_dict() for m in self.micro_batch_infos]}

    @classmethod
    def from_dict(cls, d: dict) -> "AdapterGroupStepInfo":
        return cls([MicroBatchInfo.from_dict(m) for m in d["micro_batch_infos"]])


# ----------------------------------------------------------------------------------------
# native packers
# ----------------------------------------------------------------------------------------
def _host():
    from ..ops._native import host_lib

    lib = host_lib()
    if not getattr(lib, "_lf_solver_declared", False):
        LL, I, D = C.c_longlong, C.c_int, C.c_double
        lib.lf_pack_ffd.argtypes = [C.POINTER(LL), C.POINTER(I), I, I, LL, LL, C.POINTER(I)]
        lib.lf_pack_ffd.restype = I
        lib.lf_pack_exact.argtypes = [C.POINTER(LL), C.POINTER(I), I, I, LL, LL, D, C.POINTER(I), C.POINTER(I)]
        lib.lf_pack_exact.restype = I
        lib._lf_solver_declared = True
    return lib


def _call_packer(samples: Sequence[tuple], capacity: int, pad: int, exact: bool, time_limit: float):
    """``samples`` = [(key, adapter, tokens)].  Returns (bins: list[list[key]], status)."""
    n = len(samples)
    if n == 0:
        return [], 3
    adapters = sorted({a for _, a, _ in samples})
    remap = {a: i for i, a in enumerate(adapters)}
    lens = (C.c_longlong * n)(*[int(t) for _, _, t in samples])
    ads = (C.c_int * n)(*[remap[a] for _, a, _ in samples])
    out = (C.c_int * n)()
    status = C.c_int(0)
    for _, _, t in samples:
        if _pad(int(t), pad) > capacity:
            raise ValueError(f"sample of {t} tokens does not fit a microbatch of capacity {capacity}")
    lib = _host()
    if exact:
        nb = lib.lf_pack_exact(lens, ads, n, len(adapters), capacity, pad, float(time_limit), out,
                               C.byref(status))
    else:
        nb = lib.lf_pack_ffd(lens, ads, n, len(adapters), capacity, pad, out)
    bins: list = [[] for _ in range(nb)]
    for i, (key, _, _) in enumerate(samples):
        bins[out[i]].append(key)
    return bins, status.value


def greedy_pack_decide_bins(samples: Sequence[tuple], capacity: int,
                            pad: int = ADAPTER_PADDING_MULTIPLE) -> list:
    """First-fit-decreasing packing; returns the sample keys of each bin."""
    return _call_packer(samples, capacity, pad, False, 0.0)[0]


def solve_micro_milp_lexicographic(samples: Sequence[tuple], capacity: int,
                                   pad: int = ADAPTER_PADDING_MULTIPLE, time_limit: float = 3.0):
    """Lexicographic optimum (fewest bins, then smallest leftover bin) by branch and bound
    within ``time_limit`` seconds; falls back to the best packing found.  Returns
    ``(bins, status)`` with status bits 1 = bin count proven minimal, 2 = leftover proven
    minimal, 4 = time limit hit."""
    return _call_packer(samples, capacity, pad, True, time_limit)


# ----------------------------------------------------------------------------------------
# adapter grouping
# ----------------------------------------------------------------------------------------
def estimate_microbatches(batches: Sequence[Sequence[int]], capacity: int, k_sigma: float = 0.0) -> int:
    flat = np.asarray([n for b in batches for n in b], dtype=np.float64)
    if flat.size == 0:
        return 0
    gbs = len(batches[0])
    sigma = float(flat.std(ddof=1)) if flat.size > 1 else 0.0
    return max(1, math.ceil(gbs * (float(flat.mean()) + k_sigma * sigma) / capacity))


def group_adapters(data: Sequence[Sequence[Sequence[int]]], capacity: int = 4096, *, k_sigma: float = 0.25,
                   num_stages: int = 4) -> list:
    """Head-tail pairing: adapters sorted by mean sample length, shortest paired with longest,
    as long as every group still sees at least ``num_stages - 1`` (pessimistically estimated)
    microbatches of other groups between two of its own global batches.  Returns a list of
    groups (each a list of 1 or 2 adapter indices)."""
    n = len(data)
    means = [float(np.mean([t for b in data[a] for t in b])) if data[a] else 0.0 for a in range(n)]
    order = sorted(range(n), key=lambda a: means[a])
    est = {a: estimate_microbatches(data[a], capacity, -k_sigma) for a in range(n)}

    def group_estimate(g):
        flat = [[t for a in g for t in (data[a][0] if data[a] else [])]]
        return estimate_microbatches(flat, capacity, -k_sigma) if flat[0] else 0

    def bubble_free(groups):
        ests = [group_estimate(g) for g in groups]
        total = sum(ests)
        return all(total - e >= num_stages - 1 for e in ests)

    groups = [[a] for a in order]
    lo, hi = 0, n - 1
    paired: list = []
    used = set()
    while lo < hi:
        cand = [g for g in groups if g[0] not in (order[lo], order[hi]) and g[0] not in used]
        trial = paired + [[order[lo], order[hi]]] + cand
        if bubble_free(trial) or len(trial) == 1:
            paired.append([order[lo], order[hi]])
            used.update((order[lo], order[hi]))
        lo += 1
        hi -= 1
    rest = [[a] for a in order if a not in used]
    del est
    return paired + rest


# ----------------------------------------------------------------------------------------
# packing of all (global batch, group) tasks
# ----------------------------------------------------------------------------------------
def _pack_task(task, capacity, pad, time_limit, use_exact):
    g_idx, group, samples = task
    greedy = greedy_pack_decide_bins(samples, capacity, pad)
    best = greedy
    if use_exact and len(samples) > 1:
        exact, _ = solve_micro_milp_lexicographic(samples, capacity, pad, time_limit)

        def score(bins):
            lens = {k: t for k, _, t in samples}
            ad = {k: a for k, a, _ in samples}
            loads = []
            for b in bins:
                per: dict = {}
                for k in b:
                    per[ad[k]] = per.get(ad[k], 0) + lens[k]
                loads.append(sum(_pad(v, pad) for v in per.values()))
            return (len(bins), min(loads) if loads else 0)

        if score(exact) < score(greedy):
            best = exact
    lens = {k: t for k, _, t in samples}
    infos = [MicroBatchInfo({k: lens[k] for k in b}, capacity, pad) for b in best if b]
    return g_idx, group, AdapterGroupStepInfo(infos)


def packing_data_to_microbatches_micro_milp(data, groups: Optional[list] = None, capacity: int = 4096,
                                            num_stages: int = 4, *, time_limit: float = 3.0,
                                            pad: int = ADAPTER_PADDING_MULTIPLE, use_exact: bool = True,
                                            num_workers: int = 1) -> list:
    """Pack every (global batch, adapter group) and return the schedule as a list of
    :class:`AdapterGroupStepInfo` ordered by global batch, then group."""
    if groups is None:
        groups = group_adapters(data, capacity, num_stages=num_stages)
    n_batches = max((len(d) for d in data), default=0)
    tasks = []
    for g_idx in range(n_batches):
        for group in groups:
            samples = [((a, g_idx, k), a, int(t)) for a in group if g_idx < len(data[a])
                       for k, t in enumerate(data[a][g_idx])]
            if samples:
                tasks.append((g_idx, tuple(group), samples))
    if num_workers > 1 and len(tasks) > 1:
        with ThreadPoolExecutor(num_workers) as pool:  # the native search releases the GIL
            results = list(pool.map(lambda t: _pack_task(t, capacity, pad, time_limit, use_exact), tasks))
    else:
        results = [_pack_task(t, capacity, pad, time_limit, use_exact) for t in tasks]
    return [r[2] for r in results]


def packing_data_to_microbatches_micro_milp_with_multiprocessing(data, groups=None, capacity: int = 4096,
                                                                  num_stages: int = 4, *, time_limit: float = 3.0,
                                                                  num_workers: int = 8, **kw) -> list:
    """Parallel variant (worker threads over the native search)."""
    return packing_data_to_microbatches_micro_milp(data, groups, capacity, num_stages, time_limit=time_limit,
                                                   num_workers=num_workers, **kw)


# ----------------------------------------------------------------------------------------
# bubble lemma, merge pass, verification
# ----------------------------------------------------------------------------------------
def flatten_schedule(schedule: Sequence[AdapterGroupStepInfo]) -> list:
    return [m for step in schedule for m in step.micro_batch_infos]


def bubble_lemma_violations(flat: Sequence[MicroBatchInfo], num_pipeline_stages: int) -> list:
    """Positions ``pos`` whose microbatch uses global batch ``g`` of some adapter fewer than
    ``num_pipeline_stages`` positions after the last microbatch of its batch ``g - 1`` (the
    optimizer step of ``g - 1`` would not have finished when ``g`` enters the pipeline), that
    mix two global batches of one adapter, or that return to batch ``g`` of an adapter after
    one of its later batches has already started."""
    last_pos: dict = {}
    newest: dict = {}
    bad = []
    for pos, mb in enumerate(flat):
        seen: dict = {}
        ok = True
        for a, g, _ in mb.data_samples:
            if a in seen and seen[a] != g:
                ok = False
            seen[a] = g
        for a, g in seen.items():
            prev = last_pos.get((a, g - 1))
            if prev is not None and pos - prev < num_pipeline_stages:
                ok = False
            if g < newest.get(a, g):
                ok = False  # a global batch may not resume after a later one of the same adapter began
            newest[a] = max(newest.get(a, g), g)
        if not ok:
            bad.append(pos)
        for a, g in seen.items():
            last_pos[(a, g)] = pos
    return bad


def _bubble_ok(flat, num_pipeline_stages) -> bool:
    return not bubble_lemma_violations(flat, num_pipeline_stages)


def apply_merge_pass_for_adapter_group_step_infos(schedule: list, num_pipeline_stages: int, *,
                                                  look_ahead: int = 8, delta: int = 1024,
                                                  allow_partial: bool = True) -> list:
    """Greedy tail merge with look-ahead and rollback.

    For each group step, its smallest microbatch is offered to the microbatches of the next
    ``look_ahead`` group steps (emptiest first): a full merge when everything fits, otherwise
    (``allow_partial``) a partial merge when the target has more than ``delta`` free tokens.
    A move that breaks the bubble lemma is rolled back."""
    schedule = [AdapterGroupStepInfo([MicroBatchInfo(dict(m.data_samples), m.max_microbatch_size,
                                                     m.adapter_padding_multiple, m.micro_batch_idx,
                                                     m.is_empty_marker) for m in s.micro_batch_infos])
                for s in schedule]
    for i, step in enumerate(schedule):
        if not step.micro_batch_infos:
            continue
        tail = step.micro_batch_infos[-1]
        if tail.is_empty_marker or len(step.micro_batch_infos) < 1:
            continue
        targets = [m for s in schedule[i + 1:i + 1 + look_ahead] for m in s.micro_batch_infos
                   if not m.is_empty_marker]
        targets.sort(key=lambda m: m.padded_total_tokens)
        for tgt in targets:
            if not tail.data_samples:
                break
            snap_t, snap_s = dict(tgt.data_samples), dict(tail.data_samples)
            moved = tgt.full_merge(tail)
            if not moved and allow_partial and tgt.max_microbatch_size - tgt.padded_total_tokens > delta:
                moved = tgt.partial_merge(tail) > 0
            if not moved:
                continue
            # judge the order the schedule will finally have: inside a group step the
            # microbatches are sorted by padded size, largest first
            trial = [m for s in schedule
                     for m in sorted((x for x in s.micro_batch_infos if x.data_samples or x.is_empty_marker),
                                     key=lambda x: x.padded_total_tokens, reverse=True)]
            if not _bubble_ok(trial, num_pipeline_stages):
                tgt.data_samples, tail.data_samples = snap_t, snap_s
    for s in schedule:
        s.self_update()
    return [s for s in schedule if s.micro_batch_infos]


def verify_correctness_of_schedule(data, schedule: list, num_pipeline_stages: int, *,
                                   add_bubble: bool = False):
    """Check a schedule; returns ``(ok, messages)`` -- or, with ``add_bubble``, ``(ok,
    messages, fixed_schedule)`` where empty no-op microbatches have been inserted wherever the
    bubble lemma was violated."""
    msgs = []
    flat = flatten_schedule(schedule)
    for pos, mb in enumerate(flat):
        if mb.padded_total_tokens > mb.max_microbatch_size:
            msgs.append(f"microbatch {pos}: padded size {mb.padded_total_tokens} exceeds capacity "
                        f"{mb.max_microbatch_size}")
    expected = {(a, g, k): int(t) for a, batches in enumerate(data) for g, b in enumerate(batches)
                for k, t in enumerate(b)}
    seen: dict = {}
    for pos, mb in enumerate(flat):
        for key, t in mb.data_samples.items():
            if key in seen:
                msgs.append(f"sample {key} appears in microbatches {seen[key]} and {pos}")
            seen[key] = pos
            if key not in expected:
                msgs.append(f"sample {key} is not part of the data")
            elif expected[key] != t:
                msgs.append(f"sample {key}: length {t} != {expected[key]}")
    missing = set(expected) - set(seen)
    if missing:
        msgs.append(f"{len(missing)} samples are never scheduled, e.g. {sorted(missing)[:3]}")
    for pos, mb in enumerate(flat):
        per: dict = {}
        for a, g, _ in mb.data_samples:
            per.setdefault(a, set()).add(g)
        for a, gs in per.items():
            if len(gs) > 1:
                msgs.append(f"microbatch {pos} mixes global batches {sorted(gs)} of adapter {a}")
    bad = bubble_lemma_violations(flat, num_pipeline_stages)
    if not add_bubble:
        if bad:
            msgs.append(f"bubble lemma violated at microbatch positions {bad[:8]}")
        return (not msgs), msgs
    fixed = []
    capacity = flat[0].max_microbatch_size if flat else 0
    for step in schedule:
        out = []
        for mb in step.micro_batch_infos:
            trial = flatten_schedule(fixed) + out + [mb]
            guard = 0
            while bubble_lemma_violations(trial, num_pipeline_stages) and guard < num_pipeline_stages:
                out.append(MicroBatchInfo.empty_marker(capacity))
                trial = flatten_schedule(fixed) + out + [mb]
                guard += 1
            out.append(mb)
        s = AdapterGroupStepInfo.__new__(AdapterGroupStepInfo)
        s.micro_batch_infos = out  # keep the execution order (no re-sorting)
        fixed.append(s)
    left = bubble_lemma_violations(flatten_schedule(fixed), num_pipeline_stages)
    if left:
        msgs.append(f"bubble lemma still violated at {left[:8]} after inserting no-ops")
    return (not msgs), msgs, fixed


# ----------------------------------------------------------------------------------------
# serialisation (JSON mirror + pickle, named <dataset>_cap<C>_ada<k>_pp<S>_gbz<G>)
# ----------------------------------------------------------------------------------------
def schedule_name(dataset: str, capacity: int, num_adapters: int, num_stages: int, gbs: int) -> str:
    return f"{dataset}_cap{capacity}_ada{num_adapters}_pp{num_stages}_gbz{gbs}"


def save_schedule(schedule: list, path: str | Path) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    payload = [s.to_dict() for s in schedule]
    path.with_suffix(".json").write_text(json.dumps(payload))
    with open(path.with_suffix(".pkl"), "wb") as f:
        pickle.dump(schedule, f)


def load_schedule(path: str | Path) -> list:
    path = Path(path)
    if path.suffix == ".pkl":
        with open(path, "rb") as f:
            return pickle.load(f)
    return [AdapterGroupStepInfo.from_dict(d) for d in json.loads(path.with_suffix(".json").read_text())]


def schedule_statistics(schedule: list) -> dict:
    flat = [m for m in flatten_schedule(schedule) if not m.is_empty_marker]
    if not flat:
        return {"num_microbatches": 0}
    cap = flat[0].max_microbatch_size
    real = sum(m.total_tokens for m in flat)
    padded = sum(m.padded_total_tokens for m in flat)
    return {"num_microbatches": len(flat), "num_noops": len(flatten_schedule(schedule)) - len(flat),
            "real_tokens": real, "padded_tokens": padded, "fill": real / (len(flat) * cap),
            "padding_overhead": padded / max(real, 1) - 1.0}
