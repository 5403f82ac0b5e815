"""Single-stage (no pipeline) multi-LoRA trainer: the call a user makes for DP training.

One step = every scheduled microbatch goes forward and backward through the frozen base with
all adapters batched together, LoRA gradients are reduced over the data-parallel group, and
every adapter that completed its global batch takes an AdamW step.  It plays the role of the
reference's ``standard_benchmarking`` + ``multi_lora_forward_backward_no_pipelining`` loop
(``benchmarks_paper/bench_multi_gpu.py:673-691``,
``lorafusion/pipeline_parallel/multi_lora_schedule.py:130-300``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..models.config import AdapterSpec, ModelConfig
from ..models.decoder import DecoderStage, PackedBatch
from ..utils.benchmark import nvtx_range
from .data import MicroBatchSpec, build_packed_batch, stage_host_batch


@dataclass
class OptimizerConfig:
    lr: float = 1e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0


class MultiLoRATrainer:
    def __init__(self, cfg: ModelConfig, adapters: Sequence[AdapterSpec], device, *,
                 quantize: bool = False, recompute=True, optim: Optional[OptimizerConfig] = None,
                 dp_group=None, seed: int = 0, init_b_std: float = 0.0, grad_sync: str = "auto",
                 use_multimem: bool = False, use_fsdp: bool = False):
        """``use_fsdp``: ZeRO-3 style baseline -- the frozen base is sharded over the data-parallel
        group and gathered layer by layer (``models/fsdp_decoder.py``)."""
        self.cfg = cfg
        self.adapters = list(adapters)
        self.device = torch.device(device)
        self.optim = optim or OptimizerConfig()
        self.dp_group = dp_group
        self.dp_size = dist.get_world_size(dp_group) if (dist.is_initialized() and dp_group is not None) else 1
        # grad_sync: "fused" = one reduce+Adam+broadcast kernel per adapter over NVLink peer
        # memory (default when dp > 1), "nccl" = NCCL all-reduce then the local Adam kernel
        # (the unfused baseline), "auto" = fused when dp > 1.
        self.grad_sync = ("fused" if self.dp_size > 1 else "local") if grad_sync == "auto" else grad_sync
        alloc = None
        if self.grad_sync == "fused":
            from ..parallel.symmetric import SymmetricAllocator

            alloc = SymmetricAllocator(self.device, dp_group)
        kw = dict(quantize=quantize, recompute=recompute, seed=seed, init_b_std=init_b_std, shared_alloc=alloc)
        if use_fsdp:
            from ..models.fsdp_decoder import FsdpDecoderStage

            self.stage = FsdpDecoderStage(cfg, adapters, device, dp_group if self.dp_size > 1 else None, **kw)
        else:
            self.stage = DecoderStage(cfg, adapters, device, **kw)
        self.step_count = 0
        self._fused_sync = None
        if self.grad_sync == "fused" and self.stage.arena is not None:
            from ..parallel.dp_sync import FusedGradSync

            self._fused_sync = FusedGradSync(self.stage.arena, alloc, dp_group, self.optim,
                                             use_multimem=use_multimem)

    # ------------------------------------------------------------------ data movement
    def stage_batches(self, specs: Sequence[MicroBatchSpec], seed: int) -> list:
        """Create the host-side (pinned) arrays of a step's microbatches."""
        return [stage_host_batch(s, self.cfg.vocab_size, seed * 1000 + i) for i, s in enumerate(specs)]

    def to_device(self, specs: Sequence[MicroBatchSpec], host: Sequence, seed: int) -> list[PackedBatch]:
        return [build_packed_batch(s, self.adapters, self.cfg.vocab_size, self.device, seed=seed * 1000 + i,
                                   host=h) for i, (s, h) in enumerate(zip(specs, host))]

    # ------------------------------------------------------------------ step
    def step_on_device(self, batches: Sequence[PackedBatch], active_adapters: Optional[Sequence[int]] = None):
        """Forward/backward of all microbatches + gradient reduction + optimizer steps.
        Returns the mean token loss as a device scalar (no host synchronisation)."""
        loss_sum = None
        n_tok = 0
        for b in batches:
            with nvtx_range("Forward+Backward"):
                ls = self.stage.forward_backward(b)
            loss_sum = ls if loss_sum is None else loss_sum + ls
            n_tok += b.num_loss_tokens
        with nvtx_range("Gradient sync + optimizer step"):
            self.reduce_and_step(len(batches), active_adapters)
        self.step_count += 1
        return loss_sum / max(n_tok, 1)

    def reduce_and_step(self, num_microbatches: int, active_adapters: Optional[Sequence[int]] = None) -> None:
        arena = self.stage.arena
        if arena is None:
            return
        active = range(len(self.adapters)) if active_adapters is None else active_adapters
        scale = 1.0 / (max(num_microbatches, 1) * self.dp_size)
        o = self.optim
        if self._fused_sync is not None:
            for a in active:
                self._fused_sync.reduce_and_step(a, grad_scale=scale)
            return
        if self.dp_size > 1:
            dist.all_reduce(arena.grad, group=self.dp_group)
        for a in active:
            arena.adam_step(a, lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps,
                            weight_decay=o.weight_decay, grad_scale=scale)

    def train_step(self, specs: Sequence[MicroBatchSpec], seed: int, host: Optional[Sequence] = None) -> float:
        """End-to-end step: pinned host arrays -> device, compute, loss back to the host."""
        if host is None:
            host = self.stage_batches(specs, seed)
        batches = self.to_device(specs, host, seed)
        loss = self.step_on_device(batches)
        return float(loss.item())
