"""Book-keeping for multi-adapter training: which microbatches are in flight and when each
adapter has seen its global batch and must synchronise gradients and step its optimizer.

Same responsibilities and method names as the reference's ``MultiLoRAManager``
(``lorafusion/ops/multi_lora.py:36-293``):

* a deque of at most ``num_pipeline_stages`` batch infos -- the forward pass of a pipeline
  stage uses the *newest*, the backward (and any recomputation) the *oldest* microbatch;
* per-adapter sample counters compared against ``multi_lora_global_batch_sizes``;
* ``maybe_reduce_grad_and_optimizer_step`` which fires the per-adapter gradient reduction +
  optimizer step.

What differs: the counters need no device all-reduce and no ``.item()`` (the reference does
one per adapter per microbatch, ``multi_lora.py:140-151``).  All data-parallel ranks execute
the same offline schedule, so every rank derives the same global count on the host
(``local count x dp size``); the step itself is a callback -- NCCL all-reduce + Adam kernel,
or the fused reduce+Adam kernel over NVLink.
"""

from __future__ import annotations

from collections import deque
from typing import Callable, Optional, Sequence

from ..models.config import AdapterSpec
from ..ops.batch_info import MultiLoRABatchInfo

_MANAGER: Optional["MultiLoRAManager"] = None


class MultiLoRAManager:
    def __init__(self, lora_configs: Sequence[AdapterSpec], num_pipeline_stages: int,
                 multi_lora_max_microbatch_tokens: Optional[int],
                 multi_lora_global_batch_sizes: Optional[Sequence[int]] = None, *, dp_size: int = 1):
        if multi_lora_global_batch_sizes is None:
            raise ValueError("multi_lora_global_batch_sizes is required")
        if len(multi_lora_global_batch_sizes) != len(lora_configs):
            raise ValueError(f"expected {len(lora_configs)} global batch sizes, got "
                             f"{len(multi_lora_global_batch_sizes)}")
        self.lora_configs = list(lora_configs)
        self.num_pipeline_stages = num_pipeline_stages
        self.multi_lora_max_microbatch_tokens = multi_lora_max_microbatch_tokens
        self.multi_lora_global_batch_sizes = [int(v) for v in multi_lora_global_batch_sizes]
        self.dp_size = dp_size
        self.adapter_sample_counts = {i: 0 for i in range(len(self.lora_configs))}
        self.adapter_microbatch_counts = {i: 0 for i in range(len(self.lora_configs))}
        self.batch_info_deque: deque = deque(maxlen=num_pipeline_stages)
        self.microbatch_idx = 0
        self.is_in_backward = False
        self.step_fn: Optional[Callable[[int, int], None]] = None
        self.steps_taken = {i: 0 for i in range(len(self.lora_configs))}
        self._pending_counts: deque = deque()

    # ------------------------------------------------------------------ optimizer hook
    def register_step_fn(self, fn: Callable[[int, int], None]) -> None:
        """``fn(adapter_idx, num_microbatches)`` reduces the adapter's gradients over the
        data-parallel group and applies its optimizer step."""
        self.step_fn = fn

    def register_ddp_modules_and_optimizers(self, ddp_model=None, ddp_modules=None, optimizers=None) -> None:
        """Accepted for call compatibility: gradient buffers and optimizer state live in the
        LoRA arena, so there is nothing to register besides the step function."""
        del ddp_model, ddp_modules, optimizers

    # ------------------------------------------------------------------ in-flight microbatches
    def add_batch_info(self, batch_info: MultiLoRABatchInfo) -> None:
        if len(self.batch_info_deque) == self.num_pipeline_stages:
            raise ValueError(f"more than {self.num_pipeline_stages} microbatches in flight")
        batch_info.microbatch_idx = self.microbatch_idx
        self.microbatch_idx += 1
        self.batch_info_deque.append(batch_info)
        mbi = batch_info.micro_batch_info
        if mbi is None:
            if batch_info.allow_empty_micro_batch_info:
                self._pending_counts.append({})
                return
            raise ValueError("MicroBatchInfo is not available")
        counts = {}
        if hasattr(mbi, "adapter_num_samples_pairs"):
            counts = dict(mbi.adapter_num_samples_pairs)
        elif hasattr(mbi, "segments"):
            counts = {a: len(lens) for a, lens in mbi.segments if a >= 0}
        for a in counts:
            if a not in self.adapter_sample_counts:
                raise ValueError(f"adapter {a} is unknown to the manager")
        self._pending_counts.append(counts)

    def get_newest_batch_info(self) -> Optional[MultiLoRABatchInfo]:
        return self.batch_info_deque[-1] if self.batch_info_deque else None

    def get_oldest_batch_info(self) -> Optional[MultiLoRABatchInfo]:
        return self.batch_info_deque[0] if self.batch_info_deque else None

    def get_current_batch_info(self) -> Optional[MultiLoRABatchInfo]:
        """Newest in a forward pass, oldest in a backward pass / recomputation."""
        return self.get_oldest_batch_info() if self.is_in_backward else self.get_newest_batch_info()

    def pop_oldest_batch_info(self) -> Optional[MultiLoRABatchInfo]:
        """Retire the oldest microbatch (its backward has finished) and credit its samples
        to the adapters' counters."""
        if not self.batch_info_deque:
            return None
        info = self.batch_info_deque.popleft()
        counts = self._pending_counts.popleft() if self._pending_counts else {}
        for a, n in counts.items():
            self.adapter_sample_counts[a] += n
            self.adapter_microbatch_counts[a] += 1
        return info

    def clear_batch_info(self) -> None:
        self.batch_info_deque.clear()
        self._pending_counts.clear()

    # ------------------------------------------------------------------ phase marks
    @property
    def is_in_forward(self) -> bool:
        return not self.is_in_backward

    def set_backward_pass_state(self, *, is_backward: bool) -> bool:
        self.is_in_backward = is_backward
        return True

    def mark_backward_pass_started(self) -> bool:
        return self.set_backward_pass_state(is_backward=True)

    def mark_forward_pass_started(self) -> bool:
        return self.set_backward_pass_state(is_backward=False)

    # ------------------------------------------------------------------ optimizer steps
    def maybe_reduce_grad_and_optimizer_step(self) -> list:
        """Step every adapter whose global batch is complete; returns their indices."""
        stepped = []
        for a, local in self.adapter_sample_counts.items():
            total = local * self.dp_size
            target = self.multi_lora_global_batch_sizes[a]
            if total > target:
                raise ValueError(f"adapter {a} overshot its global batch: {total} > {target}")
            if total == target and total > 0:
                self.reduce_grad_and_optimizer_step(a)
                stepped.append(a)
        return stepped

    def reduce_grad_and_optimizer_step(self, adapter_idx: int) -> None:
        if self.step_fn is None:
            raise RuntimeError("no optimizer step function registered")
        self.step_fn(adapter_idx, max(self.adapter_microbatch_counts[adapter_idx], 1))
        self.adapter_sample_counts[adapter_idx] = 0
        self.adapter_microbatch_counts[adapter_idx] = 0
        self.steps_taken[adapter_idx] += 1


def init_multi_lora_manager(lora_configs, num_pipeline_stages, multi_lora_max_microbatch_tokens,
                            multi_lora_global_batch_sizes=None, *, dp_size: int = 1,
                            replace: bool = False) -> MultiLoRAManager:
    global _MANAGER
    if _MANAGER is not None and not replace:
        raise ValueError("Multi-LoRA manager has already been initialized")
    _MANAGER = MultiLoRAManager(lora_configs, num_pipeline_stages, multi_lora_max_microbatch_tokens,
                                multi_lora_global_batch_sizes, dp_size=dp_size)
    return _MANAGER


def get_multi_lora_manager() -> Optional[MultiLoRAManager]:
    return _MANAGER


def reset_multi_lora_manager() -> None:
    global _MANAGER
    _MANAGER = None
