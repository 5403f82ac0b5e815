"""Pipeline-parallel runtime: non-interleaved 1F1B over NCCL (or gloo) point-to-point.

Replaces the reference's copies of Megatron's schedules
(``lorafusion/pipeline_parallel/multi_lora_schedule.py:130-726``) and Megatron's p2p layer:

* **No shape handshake and no empty-batch marker tensors.**  The microbatch schedule is
  produced offline, so every stage knows each microbatch's padded token count in advance and
  receive buffers are allocated directly.  Empty (no-op) microbatches -- inserted by the
  solver to satisfy the bubble lemma -- keep their SLOT in the 1F1B order on every stage: a
  no-op forward and a no-op backward advance the schedule position exactly like a real
  microbatch, but compute nothing and send nothing (the reference sends a ``(1, 1, 7)``
  marker tensor through the pipeline, ``multi_lora_schedule.py:36,560-592``).  Dropping the
  slots instead would pull the first microbatch of an adapter's next global batch forward,
  ahead of the optimizer step of the previous one.
* **The bubble lemma is asserted at run time**: before executing, :meth:`PipelineRuntime.run`
  checks that every microbatch of global batch ``g + 1`` of an adapter sits at least
  ``pp`` slots after the last microbatch of its batch ``g``, and raises
  :class:`BubbleLemmaError` otherwise (``lorafusion/solver/proposed_solver.py:617-635``).
* **Overlapped p2p.**  Forward activations and backward gradients travel on two separate
  process groups (independent communicators and streams), receives for the next microbatch
  are posted before the current one is computed, and sends are waited on lazily.
* **Per-adapter optimizer steps inside the schedule**: after each backward the manager
  retires the oldest in-flight microbatch and steps every adapter whose global batch is
  complete; the bubble lemma guarantees no in-flight microbatch still reads those weights.

A stage is anything with ``forward(batch, h_in) -> (h_out, saved)``,
``loss_and_grad(out, batch) -> (loss, dh)`` and ``backward(saved, dh, batch) -> dh_in``
(:class:`lorafusion_b200.models.decoder.DecoderStage` or a CPU toy stage in the tests).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence

import torch
import torch.distributed as dist

from .layout import ParallelState


def even_layer_partition(num_layers: int, num_stages: int) -> list:
    """``[(start, end)]`` per stage; the first ``num_layers % num_stages`` stages get one
    extra layer (``lorafusion/pipeline_parallel/pipe_module.py:98-154``)."""
    base, extra = divmod(num_layers, num_stages)
    out, start = [], 0
    for s in range(num_stages):
        n = base + (1 if s < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def get_pipeline_stage_layer_indices(num_layers: int, num_stages: int, stage_idx: int) -> list:
    s, e = even_layer_partition(num_layers, num_stages)[stage_idx]
    return list(range(s, e))


class PipeModel:
    """Factory of pipeline stages: ``PipeModel.from_model(model, stage_idx=s, num_stages=n)``
    returns the :class:`~lorafusion_b200.models.decoder.DecoderStage` that owns stage ``s``'s
    layers (embedding on the first stage, final norm + lm_head + loss on the last).

    ``model`` is either a whole-model ``DecoderStage`` -- the new stage then SHARES its frozen
    weights and copies its adapter weights, which is how a partitioned run is compared with the
    unpartitioned one -- or a ``ModelConfig``, in which case the stage is built on its own
    (random-init or NF4 weights of that architecture; every rank of a multi-GPU job does this for
    its own stage only, so no rank ever holds the whole model).  Counterpart of
    ``PipeModel.from_model`` (``lorafusion/pipeline_parallel/pipe_module.py:156-196``), which
    slices the layer list of a loaded HF model."""

    @staticmethod
    def from_model(model, *, stage_idx: int, num_stages: int, adapters=None, device=None, **stage_kwargs):
        from ..models.decoder import DecoderStage

        if isinstance(model, DecoderStage):
            cfg = model.cfg
            adapters = model.adapters if adapters is None else adapters
            device = model.device if device is None else device
        else:
            cfg = model
            if adapters is None or device is None:
                raise ValueError("building a stage from a ModelConfig needs adapters= and device=")
        if not 0 <= stage_idx < num_stages:
            raise ValueError(f"stage_idx {stage_idx} outside [0, {num_stages})")
        start, end = even_layer_partition(cfg.num_layers, num_stages)[stage_idx]
        stage = DecoderStage(cfg, adapters, device, layer_start=start, layer_end=end, **stage_kwargs)
        if isinstance(model, DecoderStage):
            stage.adopt_weights(model)
        return stage


# The reference marks a no-op microbatch by sending input ids filled with this value
# (``lorafusion/pipeline_parallel/multi_lora_schedule.py``); here the schedule is known to every
# stage, so ``PipelineMicrobatch.is_empty`` carries the information and nothing is sent.  The
# constant is kept for schedule files that use it.
EMPTY_BATCH_MAGIC_TOKEN = 7


@dataclass
class PipelineMicrobatch:
    """What one stage needs to know about a microbatch: its device batch (``None`` for an
    empty no-op) and the padded token count that fixes the activation shape.
    ``adapter_batches`` maps adapter -> global batch index for the lemma check; when it is
    ``None`` it is read from ``batch.info.micro_batch_info.data_samples`` if that exists."""

    batch: Any
    num_tokens: int
    is_empty: bool = False
    adapter_batches: Optional[dict] = None

    def lemma_samples(self) -> dict:
        """``{(adapter, global batch, 0): 1}`` in the form the solver's lemma check reads."""
        if self.is_empty:
            return {}
        if self.adapter_batches is not None:
            return {(a, g, 0): 1 for a, g in self.adapter_batches.items()}
        info = getattr(self.batch, "info", None)
        mbi = getattr(info, "micro_batch_info", None)
        return dict(getattr(mbi, "data_samples", None) or {})


class BubbleLemmaError(RuntimeError):
    """The microbatch order would let a global batch enter the pipeline before the optimizer
    step of the adapter's previous global batch has been taken on every stage."""


def check_bubble_lemma(microbatches: Sequence["PipelineMicrobatch"], num_pipeline_stages: int) -> None:
    """Raise :class:`BubbleLemmaError` if the order (no-op slots included) violates the lemma."""
    if num_pipeline_stages <= 1:
        return
    from types import SimpleNamespace

    from ..solver.schedule import bubble_lemma_violations

    flat = [SimpleNamespace(data_samples=m.lemma_samples()) for m in microbatches]
    bad = bubble_lemma_violations(flat, num_pipeline_stages)
    if bad:
        raise BubbleLemmaError(
            f"bubble lemma violated at microbatch slots {bad[:8]} for {num_pipeline_stages} pipeline stages: "
            "a global batch would start before the previous optimizer step of its adapter; insert no-op "
            "microbatches (verify_correctness_of_schedule(add_bubble=True))")


@dataclass
class PipelineStats:
    loss_sum: float = 0.0
    real_tokens: int = 0
    forward_s: float = 0.0
    backward_s: float = 0.0
    total_s: float = 0.0
    stepped: list = field(default_factory=list)

    @property
    def bubble_ratio(self) -> float:
        return 1.0 - (self.forward_s + self.backward_s) / self.total_s if self.total_s > 0 else 0.0


class _P2P:
    """Asynchronous activation / gradient exchange with the neighbouring stages."""

    def __init__(self, state: ParallelState, fwd_group, bwd_group, hidden: int, dtype, device):
        self.state, self.fwd_group, self.bwd_group = state, fwd_group, bwd_group
        self.hidden, self.dtype, self.device = hidden, dtype, device
        self._pending_sends: list = []

    def _buf(self, tokens: int) -> torch.Tensor:
        return torch.empty((tokens, self.hidden), dtype=self.dtype, device=self.device)

    def post_recv_forward(self, tokens: int):
        if self.state.is_first_stage:
            return None
        buf = self._buf(tokens)
        return buf, dist.irecv(buf, src=self.state.prev_rank, group=self.fwd_group)

    def post_recv_backward(self, tokens: int):
        if self.state.is_last_stage:
            return None
        buf = self._buf(tokens)
        return buf, dist.irecv(buf, src=self.state.next_rank, group=self.bwd_group)

    def send_forward(self, t: torch.Tensor) -> None:
        if not self.state.is_last_stage:
            self._pending_sends.append((t, dist.isend(t.contiguous(), dst=self.state.next_rank, group=self.fwd_group)))

    def send_backward(self, t: Optional[torch.Tensor]) -> None:
        if not self.state.is_first_stage and t is not None:
            self._pending_sends.append((t, dist.isend(t.contiguous(), dst=self.state.prev_rank, group=self.bwd_group)))

    @staticmethod
    def wait(handle):
        if handle is None:
            return None
        buf, req = handle
        req.wait()
        return buf

    def drain(self) -> None:
        for _, req in self._pending_sends:
            req.wait()
        self._pending_sends.clear()

    def reap(self) -> None:
        """Drop completed sends (keeps tensors alive only while in flight)."""
        self._pending_sends = [(t, r) for t, r in self._pending_sends if not r.is_completed()]


class PipelineRuntime:
    def __init__(self, stage, state: ParallelState, *, hidden_size: int, dtype=torch.bfloat16, device="cuda",
                 manager=None, fwd_group=None, bwd_group=None, use_timers: bool = False,
                 health=None, health_every: int = 1):
        """``health`` (a :class:`~lorafusion_b200.parallel.health.HealthMonitor`) is consulted
        on the host before every ``health_every``-th forward or backward slot, so that a peer
        that raised or left is noticed before the next launch instead of by a device-side
        wait running out; each consulted slot also publishes this rank's progress."""
        self.stage, self.state, self.manager = stage, state, manager
        self.device = torch.device(device)
        self.p2p = _P2P(state, fwd_group, bwd_group, hidden_size, dtype, self.device)
        self.use_timers = use_timers
        self.health, self.health_every = health, max(1, int(health_every))
        self._slot_counter = 0
        self.executed_ops: list = []  # ("F" | "B", slot index, is_empty) of the last run

    # ------------------------------------------------------------------ timing helper
    def _tick(self) -> float:
        if self.use_timers and self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        return time.perf_counter()

    # ------------------------------------------------------------------ single ops
    def _forward(self, mb: PipelineMicrobatch, recv_handle, stats: PipelineStats):
        if self.manager is not None:
            self.manager.mark_forward_pass_started()
            self.manager.add_batch_info(mb.batch.info)
        h_in = self.p2p.wait(recv_handle)
        t0 = self._tick()
        out, saved = self.stage.forward(mb.batch, h_in)
        entry = dict(saved=saved, out=None, dh=None)
        if self.state.is_last_stage:
            loss, dh = self.stage.loss_and_grad(out, mb.batch)
            entry["dh"] = dh
            stats.loss_sum = stats.loss_sum + loss
            stats.real_tokens += getattr(mb.batch, "num_real_tokens", 0)
        else:
            self.p2p.send_forward(out)
        stats.forward_s += self._tick() - t0
        return entry

    def _backward(self, mb: PipelineMicrobatch, entry, recv_handle, stats: PipelineStats):
        if self.manager is not None:
            self.manager.mark_backward_pass_started()
        dh = entry["dh"] if self.state.is_last_stage else self.p2p.wait(recv_handle)
        t0 = self._tick()
        dh_in = self.stage.backward(entry["saved"], dh, mb.batch)
        self.p2p.send_backward(dh_in)
        stats.backward_s += self._tick() - t0
        if self.manager is not None:
            self.manager.pop_oldest_batch_info()
            stats.stepped += self.manager.maybe_reduce_grad_and_optimizer_step()

    # ------------------------------------------------------------------ schedules
    def _check_health(self) -> None:
        if self.health is None:
            return
        self._slot_counter += 1
        if self._slot_counter % self.health_every == 0:
            self.health.progress()
            self.health.check()

    def run(self, microbatches: Sequence[PipelineMicrobatch]) -> PipelineStats:
        """Execute one list of microbatches with 1F1B (or plainly when there is one stage).
        Empty microbatches occupy a forward and a backward slot but do no work."""
        stats = PipelineStats()
        t_start = self._tick()
        work = list(microbatches)
        pp = self.state.layout.pp
        if self.manager is not None:  # per-adapter optimizer steps happen inside the schedule
            check_bubble_lemma(work, pp)
        M = len(work)
        warm = min(pp - self.state.pp_rank - 1, M)
        steady = M - warm
        in_flight: list = []
        self.executed_ops = []

        def next_real(idx: int) -> Optional[int]:
            """Index of the first non-empty microbatch at or after ``idx``."""
            while idx < M and work[idx].is_empty:
                idx += 1
            return idx if idx < M else None

        # One forward receive is pre-posted at any time: that of the next non-empty microbatch.
        posted_f = next_real(0)
        recv_f = self.p2p.post_recv_forward(work[posted_f].num_tokens) if posted_f is not None else None

        def forward_slot(i: int) -> None:
            nonlocal posted_f, recv_f
            self._check_health()
            self.executed_ops.append(("F", i, work[i].is_empty))
            if work[i].is_empty:
                in_flight.append(None)
                return
            assert posted_f == i
            handle = recv_f
            entry = self._forward(work[i], handle, stats)
            in_flight.append(entry)
            posted_f = next_real(i + 1)
            recv_f = self.p2p.post_recv_forward(work[posted_f].num_tokens) if posted_f is not None else None

        def backward_slot(i: int) -> None:
            self._check_health()
            self.executed_ops.append(("B", i, work[i].is_empty))
            entry = in_flight.pop(0)
            if work[i].is_empty:
                return
            recv_b = self.p2p.post_recv_backward(work[i].num_tokens)
            self._backward(work[i], entry, recv_b, stats)
            self.p2p.reap()

        nf = nb = 0  # next forward / backward slot
        for _ in range(warm):
            forward_slot(nf)
            nf += 1
        for _ in range(steady):
            forward_slot(nf)
            nf += 1
            backward_slot(nb)
            nb += 1
        for _ in range(warm):
            backward_slot(nb)
            nb += 1
        self.p2p.drain()
        if self.manager is not None:
            self.manager.clear_batch_info()
        stats.total_s = self._tick() - t_start
        return stats


def multi_lora_get_forward_backward_func(runtime: PipelineRuntime) -> Callable:
    """Returns the callable that runs a list of microbatches through this rank's stage
    (name kept from ``lorafusion/pipeline_parallel/multi_lora_schedule.py:130``)."""
    return runtime.run
