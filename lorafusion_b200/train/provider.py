"""Data providers: from per-adapter mock datasets to the ordered microbatches a rank executes.

``MockMultiLoRADataProvider`` plays the role of the reference's ``MockMultiLoRADataset`` +
``MockMultiLoRADataProvider`` (``lorafusion/train/training_utils.py:1100-1347``): it owns one
length dataset per adapter, obtains a schedule (loads a schedule file or runs the solver),
and yields, microbatch by microbatch, packed random-token batches with their block tables.
``DataProvider`` is the single-adapter counterpart (``training_utils.py:1003-1097``).
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Iterator, Optional, Sequence

from ..models.config import AdapterSpec
from ..solver import schedule as S
from .data import (NAMED_DISTRIBUTIONS, LengthDistribution, MicroBatchSpec, MockDataset, build_packed_batch,
                   stage_host_batch)


def spec_from_micro_batch_info(mbi: S.MicroBatchInfo, total_multiple: int = 128) -> MicroBatchSpec:
    spec = MicroBatchSpec(mbi.segments(), is_empty_marker=mbi.is_empty_marker, total_multiple=total_multiple)
    spec.micro_batch_info = mbi
    return spec


@dataclass
class ScheduledMicrobatch:
    spec: MicroBatchSpec
    info: S.MicroBatchInfo
    index: int

    @property
    def is_empty(self) -> bool:
        return self.info.is_empty_marker or not self.info.data_samples


class MockMultiLoRADataProvider:
    def __init__(self, adapters: Sequence[AdapterSpec], datasets: Sequence[MockDataset],
                 global_batch_sizes: Sequence[int], *, capacity: int, num_pipeline_stages: int, vocab_size: int,
                 schedule_path: Optional[str | Path] = None, num_global_batches: Optional[int] = None,
                 solver_time_limit: float = 1.0, use_exact: bool = True, dp_rank: int = 0, seed: int = 0,
                 num_workers: int = 4, total_multiple: int = 128,
                 start_global_batches: Optional[Sequence[int]] = None, index_offset: int = 0):
        """``start_global_batches[i]`` = global batches of adapter ``i`` already consumed by an
        earlier run (resume): they are skipped.  ``index_offset`` = microbatches that run
        executed; it keeps the per-microbatch seeds (token ids, dropout) going where they stopped."""
        self.total_multiple = total_multiple
        self.index_offset = int(index_offset)
        self.adapters, self.datasets = list(adapters), list(datasets)
        self.global_batch_sizes = [int(g) for g in global_batch_sizes]
        self.capacity, self.num_pipeline_stages, self.vocab_size = capacity, num_pipeline_stages, vocab_size
        self.dp_rank, self.seed = dp_rank, seed
        self.data = [ds.global_batches(g) for ds, g in zip(self.datasets, self.global_batch_sizes)]
        if start_global_batches is not None:
            self.data = [d[int(s0):] for d, s0 in zip(self.data, start_global_batches)]
        if num_global_batches is not None:
            self.data = [d[:num_global_batches] for d in self.data]
        if schedule_path is not None:
            self.schedule = S.load_schedule(schedule_path)
        else:
            groups = S.group_adapters(self.data, capacity, num_stages=num_pipeline_stages)
            packed = S.packing_data_to_microbatches_micro_milp(
                self.data, groups, capacity, num_pipeline_stages, time_limit=solver_time_limit,
                use_exact=use_exact, num_workers=num_workers)
            merged = S.apply_merge_pass_for_adapter_group_step_infos(packed, num_pipeline_stages)
            ok, msgs, fixed = S.verify_correctness_of_schedule(self.data, merged, num_pipeline_stages,
                                                               add_bubble=True)
            if not ok:
                raise RuntimeError("solver produced an invalid schedule: " + "; ".join(msgs[:3]))
            self.schedule = fixed
        self.flat = S.flatten_schedule(self.schedule)
        for i, m in enumerate(self.flat):
            m.micro_batch_idx = i
        self.processed_tokens = 0
        self.cursor = 0

    @classmethod
    def from_named_distributions(cls, adapters: Sequence[AdapterSpec], names: Sequence[str],
                                 global_batch_sizes: Sequence[int], *, num_samples: int = 256, seed: int = 0,
                                 max_len: Optional[int] = None, **kw) -> "MockMultiLoRADataProvider":
        datasets = []
        for i, name in enumerate(names):
            dist = NAMED_DISTRIBUTIONS[name]
            if max_len is not None:
                dist = LengthDistribution(dist.median, dist.sigma, dist.lo, min(dist.hi, max_len), dist.name)
            datasets.append(MockDataset.from_distribution(dist, num_samples, seed + i))
        return cls(adapters, datasets, global_batch_sizes, seed=seed, **kw)

    def __len__(self) -> int:
        return len(self.flat)

    def statistics(self) -> dict:
        return S.schedule_statistics(self.schedule)

    def microbatches(self, start: int = 0, stop: Optional[int] = None) -> list:
        stop = len(self.flat) if stop is None else min(stop, len(self.flat))
        return [ScheduledMicrobatch(spec_from_micro_batch_info(m, self.total_multiple), m, i + self.index_offset)
                for i, m in enumerate(self.flat)
                if start <= i < stop]

    def stage(self, mb: ScheduledMicrobatch):
        """Pinned host arrays of a microbatch (token ids differ per data-parallel rank)."""
        if mb.is_empty:
            return None
        return stage_host_batch(mb.spec, self.vocab_size, self.seed * 100003 + mb.index * 131 + self.dp_rank)

    def to_device(self, mb: ScheduledMicrobatch, device, host=None):
        if mb.is_empty:
            return None
        host = host if host is not None else self.stage(mb)
        batch = build_packed_batch(mb.spec, self.adapters, self.vocab_size, device,
                                   seed=self.seed * 100003 + mb.index, host=host)
        batch.info.micro_batch_info = mb.info
        return batch

    def next_batch(self, device):
        """Sequential access (reference API): the next non-consumed microbatch on ``device``."""
        mb = self.microbatches(self.cursor, self.cursor + 1)[0]
        self.cursor += 1
        self.processed_tokens += mb.info.total_tokens
        return mb, self.to_device(mb, device)


class DataProvider:
    """Single-adapter provider: fixed number of samples per microbatch, packed."""

    def __init__(self, adapter: AdapterSpec, dataset: MockDataset, *, capacity: int, vocab_size: int,
                 dp_rank: int = 0, dp_size: int = 1, seed: int = 0):
        self.adapter, self.dataset = adapter, dataset
        self.capacity, self.vocab_size = capacity, vocab_size
        self.dp_rank, self.dp_size, self.seed = dp_rank, dp_size, seed
        self.cursor = dp_rank
        self.processed_tokens = 0

    def next_spec(self) -> MicroBatchSpec:
        lens: list = []
        while True:
            n = self.dataset.lengths[self.cursor % len(self.dataset)]
            padded = ((sum(lens) + n + 127) // 128) * 128
            if lens and padded > self.capacity:
                break
            lens.append(min(n, self.capacity))
            self.cursor += self.dp_size
            if padded >= self.capacity:
                break
        self.processed_tokens += sum(lens)
        return MicroBatchSpec([(0, lens)])

    def next_batch(self, device):
        spec = self.next_spec()
        return build_packed_batch(spec, [self.adapter], self.vocab_size, device, seed=self.seed + self.cursor)
