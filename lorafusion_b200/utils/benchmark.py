"""Timing harness: CUDA events or wall clock, eager or CUDA-graph replay, L2 flushing, NVTX
ranges and a torch.profiler context.

Mirrors the reference's ``benchmark()`` / ``set_warmup_and_number`` /
``create_profiler_context`` / ``tabulate_2d_benchmark_results`` helpers
(``lorafusion/utils/benchmark.py:74-196,772-863``) with the timing rules used throughout
this repository: at least three warm-up iterations, device-side timing on the launching
stream with a synchronize on both sides, and either inputs larger than L2 or an explicit L2
flush between iterations.
"""

from __future__ import annotations

import contextlib
import csv
import statistics
import time
from pathlib import Path
from typing import Callable, Optional, Sequence

import torch

_WARMUP = 5
_NUMBER = 20
L2_BYTES = 126 * 1024 * 1024


def set_warmup_and_number(warmup: int, number: int) -> None:
    global _WARMUP, _NUMBER
    _WARMUP, _NUMBER = max(3, warmup), max(1, number)


_FLUSH_BUF: dict = {}


def flush_l2(device=None) -> None:
    """Overwrite a buffer twice the size of L2 so the next kernel starts with a cold cache."""
    device = torch.device(device or "cuda")
    buf = _FLUSH_BUF.get(device)
    if buf is None:
        buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)
        _FLUSH_BUF[device] = buf
    buf.zero_()


def benchmark(func: Callable, prepare_func: Optional[Callable] = None, *, use_cuda_graph: bool = False,
              use_cuda_event: bool = True, warmup: Optional[int] = None, number: Optional[int] = None,
              flush: bool = False, profile: bool = False, msg: str = "", reduce: str = "median") -> float:
    """Time ``func(*prepare_func())`` and return seconds per call (median by default)."""
    warmup = _WARMUP if warmup is None else max(3, warmup)
    number = _NUMBER if number is None else number
    args = prepare_func() if prepare_func is not None else ()
    if not isinstance(args, (tuple, list)):
        args = (args,)
    cuda = torch.cuda.is_available()
    run = lambda: func(*args)  # noqa: E731
    graph = None
    if use_cuda_graph and cuda:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                run()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            run()
        run = graph.replay
    for _ in range(warmup):
        run()
    if cuda:
        torch.cuda.synchronize()
    times = []
    ctx = create_profiler_context(enabled=profile)
    with ctx:
        for _ in range(number):
            if flush and cuda:
                flush_l2()
            if use_cuda_event and cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                run()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1) / 1e3)
            else:
                if cuda:
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
                run()
                if cuda:
                    torch.cuda.synchronize()
                times.append(time.perf_counter() - t0)
    val = {"median": statistics.median, "mean": statistics.fmean, "min": min}[reduce](times)
    if msg:
        print(f"{msg}: {val * 1e3:.4f} ms")
    return val


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range for filtering in Nsight tools (the reference marks RawLoRA / FusedLoRA /
    FusedMultiLoRA regions the same way, ``benchmarks_paper/bench_lora_kernels.py:323-610``)."""
    pushed = False
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        pushed = True
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()


def create_profiler_context(enabled: bool = True, output_dir: str = "./profiling-results", *, skip_first: int = 0,
                            wait: int = 0, warmup: int = 1, active: int = 3, scheduled: bool = True):
    """torch.profiler (CPU + CUDA) with a Chrome/TensorBoard trace handler, or a no-op.
    ``scheduled=False`` records everything inside the ``with`` block (no ``step()`` calls
    needed) and writes the trace on exit."""
    if not enabled:
        return contextlib.nullcontext()
    from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler

    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    if not scheduled:
        return profile(activities=acts, on_trace_ready=tensorboard_trace_handler(output_dir))
    return profile(activities=acts, schedule=schedule(skip_first=skip_first, wait=wait, warmup=warmup, active=active),
                   on_trace_ready=tensorboard_trace_handler(output_dir), record_shapes=True)


def tabulate_2d_benchmark_results(rows: Sequence[str], cols: Sequence[str], values, *, fmt: str = "{:.4f}",
                                  csv_path: Optional[str] = None, title: str = "") -> str:
    """Pretty table (and optional CSV append) of ``values[row][col]``."""
    from tabulate import tabulate

    table = [[r] + [fmt.format(values[i][j]) if values[i][j] is not None else "-" for j in range(len(cols))]
             for i, r in enumerate(rows)]
    text = tabulate(table, headers=[title] + list(cols), tablefmt="github")
    if csv_path:
        p = Path(csv_path)
        p.parent.mkdir(parents=True, exist_ok=True)
        new = not p.exists()
        with open(p, "a", newline="") as f:
            w = csv.writer(f)
            if new:
                w.writerow(["Shape"] + list(cols))
            for i, r in enumerate(rows):
                w.writerow([r] + [values[i][j] for j in range(len(cols))])
    return text


class Timers:
    """Named accumulating timers (CUDA-synchronised), the small counterpart of Megatron's
    ``Timers`` the reference uses for forward-compute / backward-compute / optimizer-step
    (``lorafusion/train/training_utils.py:79-91``)."""

    def __init__(self, sync: bool = True):
        self.sync = sync
        self.totals: dict[str, float] = {}
        self.counts: dict[str, int] = {}
        self._open: dict[str, float] = {}

    def start(self, name: str) -> None:
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        self._open[name] = time.perf_counter()

    def stop(self, name: str) -> float:
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - self._open.pop(name)
        self.totals[name] = self.totals.get(name, 0.0) + dt
        self.counts[name] = self.counts.get(name, 0) + 1
        return dt

    @contextlib.contextmanager
    def __call__(self, name: str):
        self.start(name)
        try:
            yield
        finally:
            self.stop(name)

    def summary(self) -> dict:
        return {k: {"total_s": v, "count": self.counts[k], "mean_ms": 1e3 * v / self.counts[k]}
                for k, v in self.totals.items()}
