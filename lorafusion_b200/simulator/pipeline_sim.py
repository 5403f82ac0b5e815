"""Event-driven timing simulator of non-interleaved 1F1B pipelines and baseline schedule
generators, used to study load imbalance between microbatches.

Counterpart of ``benchmarks_paper/imbalance_simulator/main_random_data.py:15-804`` and
``main_with_datasets.py:41-120``: random data generation, the 1F1B timing recurrence
(C++ core, ``csrc/solver/packer.cpp``), overlap / ordering validators, and the naive,
sorted, mLoRA-style and solver-produced schedules to compare.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import numpy as np

from ..solver import schedule as S


def generate_data(num_adapters: int, num_global_batches: int, global_batch_size: int, *,
                  distribution: str = "lognormal", median: Sequence[float] | float = 512.0,
                  sigma: Sequence[float] | float = 0.6, lo: int = 32, hi: int = 4096,
                  constant: int = 1024, seed: int = 0) -> list:
    """``data[adapter][global_batch][sample] = tokens`` from a lognormal or constant law."""
    rng = np.random.default_rng(seed)
    out = []
    for a in range(num_adapters):
        med = median[a % len(median)] if isinstance(median, (list, tuple)) else median
        sig = sigma[a % len(sigma)] if isinstance(sigma, (list, tuple)) else sigma
        batches = []
        for _ in range(num_global_batches):
            if distribution == "constant":
                lens = np.full(global_batch_size, constant)
            else:
                lens = np.clip(np.rint(rng.lognormal(np.log(med), sig, global_batch_size)), lo, hi)
            batches.append([int(v) for v in lens])
        out.append(batches)
    return out


@dataclass
class PipelineTimeline:
    f_start: np.ndarray  # [M, S]
    f_end: np.ndarray
    b_start: np.ndarray
    b_end: np.ndarray
    total_time: float
    bubble_ratio: float

    def adjusted_bubble_ratio(self) -> float:
        """Bubble ratio after removing the unavoidable fill/drain triangle of an ideal
        balanced pipeline with the same average op time."""
        M, S = self.f_start.shape
        ideal = (S - 1) / (M + S - 1) if M > 0 else 0.0
        return max(0.0, self.bubble_ratio - ideal)


def _lib():
    from ..ops._native import host_lib

    lib = host_lib()
    if not getattr(lib, "_lf_sim_declared", False):
        D, I = C.c_double, C.c_int
        P = C.POINTER(D)
        lib.lf_simulate_1f1b.argtypes = [P, P, I, I, P, P, P, P, P]
        lib.lf_simulate_1f1b.restype = D
        lib._lf_sim_declared = True
    return lib


def simulate_1f1b(fwd: np.ndarray, bwd: np.ndarray) -> PipelineTimeline:
    """``fwd`` / ``bwd``: ``[M microbatches, S stages]`` durations."""
    fwd = np.ascontiguousarray(fwd, dtype=np.float64)
    bwd = np.ascontiguousarray(bwd, dtype=np.float64)
    M, Sg = fwd.shape
    outs = [np.zeros((M, Sg), dtype=np.float64) for _ in range(4)]
    ratio = C.c_double(0.0)
    P = C.POINTER(C.c_double)
    total = _lib().lf_simulate_1f1b(fwd.ctypes.data_as(P), bwd.ctypes.data_as(P), M, Sg,
                                    *[o.ctypes.data_as(P) for o in outs], C.byref(ratio))
    if total < 0:
        raise RuntimeError("inconsistent pipeline schedule")
    return PipelineTimeline(*outs, float(total), float(ratio.value))


def default_time_model(fwd_per_token: float = 1.0, bwd_ratio: float = 2.0, fixed: float = 0.0):
    """Linear op-time model: forward = fixed + tokens * fwd_per_token; backward = ratio * it."""
    def model(tokens: int, stage: int, num_stages: int):
        f = fixed + tokens * fwd_per_token / num_stages
        return f, bwd_ratio * f
    return model


def evaluate_schedule_pipeline_parallelism(microbatch_tokens: Sequence[int], num_stages: int,
                                           time_model: Optional[Callable] = None) -> PipelineTimeline:
    """Simulate a flat list of microbatches (padded token counts; 0 = empty no-op)."""
    time_model = time_model or default_time_model()
    M = len(microbatch_tokens)
    fwd = np.zeros((M, num_stages))
    bwd = np.zeros((M, num_stages))
    for m, t in enumerate(microbatch_tokens):
        for s in range(num_stages):
            fwd[m, s], bwd[m, s] = time_model(int(t), s, num_stages) if t > 0 else (0.0, 0.0)
    return simulate_1f1b(fwd, bwd)


def find_overlaps(tl: PipelineTimeline, eps: float = 1e-9) -> list:
    """Pairs of ops on the same stage whose time intervals overlap (must be empty)."""
    M, Sg = tl.f_start.shape
    bad = []
    for s in range(Sg):
        ivs = sorted([(tl.f_start[m, s], tl.f_end[m, s], "F", m) for m in range(M)] +
                     [(tl.b_start[m, s], tl.b_end[m, s], "B", m) for m in range(M)])
        for (s0, e0, k0, m0), (s1, e1, k1, m1) in zip(ivs, ivs[1:]):
            if s1 < e0 - eps:
                bad.append((s, (k0, m0), (k1, m1)))
    return bad


def check_forward_backward_constraints(tl: PipelineTimeline, eps: float = 1e-9) -> list:
    """Dependency violations: F(m, s) after F(m, s-1); B(m, s) after B(m, s+1) and F(m, s)."""
    M, Sg = tl.f_start.shape
    bad = []
    for m in range(M):
        for s in range(Sg):
            if s > 0 and tl.f_start[m, s] < tl.f_end[m, s - 1] - eps:
                bad.append(("F", m, s))
            if s < Sg - 1 and tl.b_start[m, s] < tl.b_end[m, s + 1] - eps:
                bad.append(("B", m, s))
            if tl.b_start[m, s] < tl.f_end[m, s] - eps:
                bad.append(("FB", m, s))
    return bad


# ----------------------------------------------------------------------------------------
# baseline schedules
# ----------------------------------------------------------------------------------------
def generate_naive_schedule(data, capacity: int, *, interleave_adapters: bool = False) -> list:
    """One adapter at a time, samples in arrival order, a new microbatch whenever the next
    sample would overflow the capacity (what per-job Megatron-style training does).  With
    ``interleave_adapters`` the global batches of the adapters alternate."""
    n_batches = max(len(d) for d in data)
    order = [(a, g) for g in range(n_batches) for a in range(len(data)) if g < len(data[a])] \
        if interleave_adapters else [(a, g) for a in range(len(data)) for g in range(len(data[a]))]
    sched = []
    for a, g in order:
        infos, cur = [], {}
        for k, t in enumerate(data[a][g]):
            trial = dict(cur)
            trial[(a, g, k)] = t
            if cur and S.MicroBatchInfo(trial, capacity).padded_total_tokens > capacity:
                infos.append(S.MicroBatchInfo(cur, capacity))
                cur = {(a, g, k): t}
            else:
                cur = trial
        if cur:
            infos.append(S.MicroBatchInfo(cur, capacity))
        step = S.AdapterGroupStepInfo.__new__(S.AdapterGroupStepInfo)
        step.micro_batch_infos = infos
        sched.append(step)
    return sched


def generate_sorted_schedule(data, capacity: int) -> list:
    """Like the naive schedule but each global batch is packed first-fit-decreasing."""
    sched = []
    for a in range(len(data)):
        for g, batch in enumerate(data[a]):
            samples = [((a, g, k), a, int(t)) for k, t in enumerate(batch)]
            bins = S.greedy_pack_decide_bins(samples, capacity)
            lens = {k: t for k, _, t in samples}
            sched.append(S.AdapterGroupStepInfo([S.MicroBatchInfo({k: lens[k] for k in b}, capacity)
                                                 for b in bins]))
    return sched


def generate_mlora_schedule(data, capacity: int) -> list:
    """mLoRA-style batching: microbatch ``i`` takes sample ``i`` of every adapter (adapters
    are concatenated in one microbatch, no bin packing); samples that do not fit spill into
    an extra microbatch."""
    n_batches = max(len(d) for d in data)
    sched = []
    for g in range(n_batches):
        infos = []
        gbs = max(len(data[a][g]) for a in range(len(data)) if g < len(data[a]))
        for k in range(gbs):
            cur = {}
            for a in range(len(data)):
                if g < len(data[a]) and k < len(data[a][g]):
                    trial = dict(cur)
                    trial[(a, g, k)] = data[a][g][k]
                    if cur and S.MicroBatchInfo(trial, capacity).padded_total_tokens > capacity:
                        infos.append(S.MicroBatchInfo(cur, capacity))
                        cur = {(a, g, k): data[a][g][k]}
                    else:
                        cur = trial
            if cur:
                infos.append(S.MicroBatchInfo(cur, capacity))
        step = S.AdapterGroupStepInfo.__new__(S.AdapterGroupStepInfo)
        step.micro_batch_infos = infos
        sched.append(step)
    return sched


def compare_schedules(data, capacity: int, num_stages: int, *, time_limit: float = 0.5,
                      time_model: Optional[Callable] = None) -> dict:
    """Simulated makespan / bubble ratio / microbatch count of the four schedule families."""
    families = {
        "naive": generate_naive_schedule(data, capacity),
        "sorted": generate_sorted_schedule(data, capacity),
        "mlora": generate_mlora_schedule(data, capacity),
    }
    groups = S.group_adapters(data, capacity, num_stages=num_stages)
    packed = S.packing_data_to_microbatches_micro_milp(data, groups, capacity, num_stages, time_limit=time_limit)
    merged = S.apply_merge_pass_for_adapter_group_step_infos(packed, num_stages)
    families["solver"] = merged
    out = {}
    for name, sched in families.items():
        # every family pays for the bubble lemma: an adapter's next global batch may only
        # enter the pipeline once the optimizer step of the previous one is done
        _, _, sched = S.verify_correctness_of_schedule(data, sched, num_stages, add_bubble=True)
        toks = [m.padded_total_tokens for m in S.flatten_schedule(sched)]
        tl = evaluate_schedule_pipeline_parallelism(toks, num_stages, time_model)
        real = sum(m.total_tokens for m in S.flatten_schedule(sched))
        out[name] = {"microbatches": len(toks), "noops": sum(1 for t in toks if t == 0), "total_time": tl.total_time, "bubble_ratio": tl.bubble_ratio,
                     "adjusted_bubble_ratio": tl.adjusted_bubble_ratio(),
                     "tokens_per_time": real / tl.total_time if tl.total_time > 0 else 0.0}
    return out


# ----------------------------------------------------------------------------------------
# latency-minimising order of a set of microbatches
# ----------------------------------------------------------------------------------------
@dataclass
class OrderSolution:
    order: list            # permutation of the input indices
    total_time: float
    bubble_ratio: float
    method: str            # "exact" or "local-search"
    evaluated: int         # simulated orders


def solve_schedule_order(microbatch_tokens: Sequence[int], num_stages: int, *,
                         time_model: Optional[Callable] = None, precedence: Sequence[tuple] = (),
                         exact_limit: int = 8, time_limit: float = 1.0, seed: int = 0) -> OrderSolution:
    """Order the microbatches so that the simulated 1F1B run finishes earliest.

    The reference states this as a MILP over forward / backward start and end times of every
    (stage, microbatch) pair (``benchmarks_paper/imbalance_simulator/proposed_solver.py:15-245``,
    solved with CBC).  Here the event-driven simulator is the objective: all orders are tried
    when there are at most ``exact_limit`` microbatches, otherwise a local search (swaps and
    re-insertions from several sorted starting points) runs until ``time_limit`` seconds.
    ``precedence`` holds ``(i, j)`` pairs meaning microbatch ``i`` must come before ``j``
    (microbatches of consecutive global batches of one adapter)."""
    import itertools
    import random
    import time as _time

    tokens = [int(t) for t in microbatch_tokens]
    M = len(tokens)
    model = time_model or default_time_model()
    fwd = np.zeros((M, num_stages))
    bwd = np.zeros((M, num_stages))
    for m, t in enumerate(tokens):
        for s in range(num_stages):
            fwd[m, s], bwd[m, s] = model(t, s, num_stages) if t > 0 else (0.0, 0.0)
    prec = [(int(i), int(j)) for i, j in precedence]
    count = 0

    def feasible(order) -> bool:
        if not prec:
            return True
        pos = {m: k for k, m in enumerate(order)}
        return all(pos[i] < pos[j] for i, j in prec)

    def cost(order) -> float:
        nonlocal count
        count += 1
        idx = list(order)
        return simulate_1f1b(fwd[idx], bwd[idx]).total_time

    if M == 0:
        return OrderSolution([], 0.0, 0.0, "exact", 0)
    if M <= exact_limit:
        best, best_c = None, float("inf")
        for perm in itertools.permutations(range(M)):
            if feasible(perm):
                c = cost(perm)
                if c < best_c - 1e-12:
                    best, best_c = list(perm), c
        if best is None:
            raise ValueError("the precedence constraints admit no order")
        tl = simulate_1f1b(fwd[best], bwd[best])
        return OrderSolution(best, tl.total_time, tl.bubble_ratio, "exact", count)

    # local search
    rng = random.Random(seed)
    asc = sorted(range(M), key=lambda m: tokens[m])
    desc = asc[::-1]
    # small ones first to fill the pipeline quickly, large ones in the middle, small ones to drain
    pyramid = asc[0::2] + asc[1::2][::-1]
    starts = [list(range(M)), desc, asc, pyramid]
    cands = [(cost(o), o) for o in starts if feasible(o)]
    if not cands:
        raise ValueError("no feasible starting order; relax the precedence constraints")
    best_c, best = min(cands, key=lambda x: x[0])
    best = list(best)
    deadline = _time.monotonic() + time_limit
    while _time.monotonic() < deadline:
        i, j = rng.randrange(M), rng.randrange(M)
        if i == j:
            continue
        trial = list(best)
        if rng.random() < 0.5:
            trial[i], trial[j] = trial[j], trial[i]
        else:
            trial.insert(j, trial.pop(i))
        if not feasible(trial):
            continue
        c = cost(trial)
        if c < best_c - 1e-12:
            best, best_c = trial, c
    tl = simulate_1f1b(fwd[best], bwd[best])
    return OrderSolution(best, tl.total_time, tl.bubble_ratio, "local-search", count)
