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


class _OverlappedSync:
    """Launches the fused reduce-scatter + AdamW + all-gather kernel per layer group on the
    trainer's side stream while the last microbatch's backward is still running below that
    group.  Every data-parallel rank creates the same groups in the same order."""

    def __init__(self, trainer: "MultiLoRATrainer", adapters: list, grad_scale: float):
        self.t, self.adapters, self.grad_scale = trainer, adapters, grad_scale
        st = trainer.stage
        n, g = len(st.layers), trainer.sync_layer_groups
        cuts = [st.layer_start + (n * k) // g for k in range(g + 1)]
        self.groups = [(cuts[k], cuts[k + 1]) for k in range(g)]     # ascending layer ranges
        self.steps = {a: trainer._fused_sync.begin_step(a) for a in adapters}
        self.launched = 0

    def on_layer_done(self, layer: int) -> None:
        # the backward walks the layers downwards: group k is complete once its lowest layer is done
        k = len(self.groups) - 1 - self.launched
        if k >= 0 and layer == self.groups[k][0]:
            self._launch(self.groups[k])
            self.launched += 1

    def _launch(self, layers: tuple) -> None:
        t = self.t
        done = torch.cuda.Event()
        done.record()                              # this group's gradients are complete here
        t._sync_stream.wait_event(done)
        with torch.cuda.stream(t._sync_stream):
            if t.tp_size > 1:   # partial sums of the replicated LoRA factors of this group, over the tp pair
                t.stage.reduce_replicated_grads(layers=layers)
            for a in self.adapters:
                t._fused_sync.reduce_and_step(a, grad_scale=self.grad_scale, layers=layers, step=self.steps[a])

    def finish(self) -> None:
        """All groups are launched; the compute stream waits for the new weights."""
        while self.launched < len(self.groups):    # a stage whose backward skipped the hook
            self._launch(self.groups[len(self.groups) - 1 - self.launched])
            self.launched += 1
        ev = torch.cuda.Event()
        ev.record(self.t._sync_stream)
        torch.cuda.current_stream(self.t.device).wait_event(ev)


class MultiLoRATrainer:
    def __init__(self, cfg: ModelConfig, adapters: Sequence[AdapterSpec], device, *,
                 quantize: bool = False, recompute=True, optim: Optional[OptimizerConfig] = None,
                 dp_group=None, seed: int = 0, init_b_std: float = 0.0, grad_sync: str = "auto",
                 use_multimem: bool = False, use_fsdp: bool = False, tp_group=None, max_tokens: int = 16384):
        """``use_fsdp``: ZeRO-3 style baseline -- the frozen base is sharded over the data-parallel
        group and gathered layer by layer (``models/fsdp_decoder.py``).
        ``tp_group``: shard every layer over this tensor-parallel group (fused all-gather -> GEMM /
        GEMM -> reduce-scatter kernels, token-sharded activations; ``models/tp_decoder.py``);
        ``dp_group`` then holds the ranks with the same position in their tensor-parallel groups,
        and all ranks of a tensor-parallel group must be given the same microbatches
        (``max_tokens`` = the largest one, a multiple of 128 x tp)."""
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
        self.tp_group = tp_group
        self.tp_size = dist.get_world_size(tp_group) if (dist.is_initialized() and tp_group is not None) else 1
        if self.tp_size > 1:
            if use_fsdp:
                raise ValueError("use_fsdp and tensor parallelism cannot be combined")
            from ..models.tp_decoder import TpDecoderStage

            self.stage = TpDecoderStage(cfg, adapters, device, tp_group, max_tokens=max_tokens, **kw)
        elif use_fsdp:
            from ..models.fsdp_decoder import FsdpDecoderStage

            self.stage = FsdpDecoderStage(cfg, adapters, device, dp_group if self.dp_size > 1 else None, **kw)
        else:
            self.stage = DecoderStage(cfg, adapters, device, **kw)
        self.step_count = 0
        # Gradient sync + optimizer step of a layer group start on a side stream as soon as the
        # last microbatch's backward has passed those layers, next to the remaining backward.
        self.sync_layer_groups = 4
        self.overlap_grad_sync = True
        self._sync_stream = None
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
        overlap = self._overlap_plan(len(batches), active_adapters)
        for i, b in enumerate(batches):
            hook = overlap.on_layer_done if (overlap is not None and i == len(batches) - 1) else None
            with nvtx_range("Forward+Backward"):
                ls = self.stage.forward_backward(b, on_layer_done=hook)
            loss_sum = ls if loss_sum is None else loss_sum + ls
            n_tok += b.num_loss_tokens
        with nvtx_range("Gradient sync + optimizer step"):
            if overlap is not None:
                overlap.finish()
            else:
                self.reduce_and_step(len(batches), active_adapters)
        self.step_count += 1
        return loss_sum / max(n_tok, 1)

    def _overlap_plan(self, num_microbatches: int, active_adapters):
        """The layer-group launcher of this step, or None when the sync runs after the backward
        (no fused kernel, overlap switched off, or a stage with too few layers to split)."""
        n_layers = len(self.stage.layers)
        if self._fused_sync is None or not self.overlap_grad_sync or n_layers < 2 * self.sync_layer_groups:
            return None
        if self.tp_size > 1:
            # Under tensor parallelism the compute stream's own kernels wait on a peer (the fused
            # all-gather -> GEMM / GEMM -> reduce-scatter kernels).  A sync kernel spinning on a side
            # stream can then hold the SMs a GEMM of this GPU needs while the rank it waits for is
            # itself behind a GEMM that waits for this GPU: a cycle over the four ranks of two
            # replicas that only the bounded waits break (seen once as "timeout waiting for a TMA
            # stage" on 4 GPUs).  Kernels that wait on other GPUs are kept in ONE stream order.
            return None
        if self._sync_stream is None:
            self._sync_stream = torch.cuda.Stream(self.device)
        active = list(range(len(self.adapters)) if active_adapters is None else active_adapters)
        return _OverlappedSync(self, active, 1.0 / (max(num_microbatches, 1) * self.dp_size))

    def reduce_and_step(self, num_microbatches: int, active_adapters: Optional[Sequence[int]] = None) -> None:
        arena = self.stage.arena
        if arena is None:
            return
        active = range(len(self.adapters)) if active_adapters is None else active_adapters
        scale = 1.0 / (max(num_microbatches, 1) * self.dp_size)
        o = self.optim
        if self.tp_size > 1:
            self.stage.reduce_replicated_grads()   # partial sums of the replicated factors, every adapter
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
