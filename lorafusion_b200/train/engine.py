"""dp x pp x tp training engine: builds this rank's stage, wires the pipeline runtime, the
multi-LoRA manager and the gradient synchronisation, and runs solver schedules.

It is the counterpart of ``setup_model_and_optimizer`` + ``standard_benchmarking`` in the
reference's multi-GPU driver (``benchmarks_paper/bench_multi_gpu.py:242-291,538-691``), with
tensor parallelism added and Megatron replaced by the runtime of ``lorafusion_b200.parallel``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..models.config import AdapterSpec, ModelConfig
from ..models.decoder import DecoderStage
from ..parallel.layout import ParallelLayout, ParallelState, initialize_parallel_state
from ..parallel.pipeline import PipelineMicrobatch, PipelineRuntime, PipelineStats, even_layer_partition
from .manager import MultiLoRAManager
from .provider import MockMultiLoRADataProvider
from .trainer import OptimizerConfig


@dataclass
class EngineConfig:
    layout: str = "dp1"
    quantize: bool = False
    recompute: object = True            # True | False | "auto"
    grad_sync: str = "auto"             # auto | fused | nccl
    capacity: int = 16384
    seed: int = 0
    init_b_std: float = 0.0
    use_timers: bool = False
    use_fsdp: bool = False              # ZeRO-3 style baseline: base weights sharded over dp


class ParallelTrainer:
    def __init__(self, cfg: ModelConfig, adapters: Sequence[AdapterSpec], global_batch_sizes: Sequence[int],
                 device, engine: EngineConfig, optim: Optional[OptimizerConfig] = None, health=None):
        """``health``: optional :class:`~lorafusion_b200.parallel.health.HealthMonitor`; the
        pipeline runtime consults it between microbatch slots."""
        self.cfg, self.adapters, self.engine = cfg, list(adapters), engine
        self.device = torch.device(device)
        self.optim = optim or OptimizerConfig()
        world = dist.get_world_size() if dist.is_initialized() else 1
        self.layout = ParallelLayout.parse(engine.layout, world)
        if world > 1:
            self.state: ParallelState = initialize_parallel_state(self.layout)
            pp_ranks = self.layout.pp_group_ranks(self.state.rank)
            self.fwd_group = self.bwd_group = None
            for ranks in self.layout.all_groups("pp"):
                if len(ranks) > 1:
                    f, b = dist.new_group(ranks), dist.new_group(ranks)
                    if ranks == pp_ranks:
                        self.fwd_group, self.bwd_group = f, b
        else:
            self.state = ParallelState(self.layout, 0, 0, 0, 0)
            self.fwd_group = self.bwd_group = None
        st = self.state
        l0, l1 = even_layer_partition(cfg.num_layers, self.layout.pp)[st.pp_rank]
        grad_sync = engine.grad_sync
        if grad_sync == "auto":
            grad_sync = "fused" if self.layout.dp > 1 else "local"
        self.grad_sync = grad_sync
        alloc = None
        if grad_sync == "fused":
            from ..parallel.symmetric import SymmetricAllocator

            alloc = SymmetricAllocator(self.device, st.dp_group)
        kw = dict(layer_start=l0, layer_end=l1, quantize=engine.quantize, recompute=engine.recompute,
                  seed=engine.seed, init_b_std=engine.init_b_std, shared_alloc=alloc,
                  max_inflight=self.layout.pp - st.pp_rank)
        if self.layout.tp > 1:
            if engine.use_fsdp:
                raise ValueError("use_fsdp and tensor parallelism cannot be combined")
            from ..models.tp_decoder import TpDecoderStage

            self.stage = TpDecoderStage(cfg, adapters, self.device, st.tp_group, max_tokens=engine.capacity, **kw)
        elif engine.use_fsdp:
            if self.layout.pp > 1:
                raise ValueError("use_fsdp shards the base over the data-parallel group of an unpartitioned model: "
                                 "pipeline_parallel_size must be 1 (the reference's FSDP arm has no pipeline either)")
            from ..models.fsdp_decoder import FsdpDecoderStage

            self.stage = FsdpDecoderStage(cfg, adapters, self.device, st.dp_group if self.layout.dp > 1 else None, **kw)
            if engine.recompute == "auto":
                self.stage.plan_activations(engine.capacity)
        else:
            self.stage = DecoderStage(cfg, adapters, self.device, **kw)
            if engine.recompute == "auto":
                self.stage.plan_activations(engine.capacity)
        self._fused = None
        if grad_sync == "fused":
            from ..parallel.dp_sync import FusedGradSync

            self._fused = FusedGradSync(self.stage.arena, alloc, st.dp_group, self.optim)
        self.manager = MultiLoRAManager(adapters, self.layout.pp, engine.capacity, global_batch_sizes,
                                        dp_size=self.layout.dp)
        self.manager.register_step_fn(self._step_adapter)
        self.runtime = PipelineRuntime(self.stage, st, hidden_size=cfg.hidden_size, device=self.device,
                                       manager=self.manager, fwd_group=self.fwd_group, bwd_group=self.bwd_group,
                                       use_timers=engine.use_timers, health=health)

    # ------------------------------------------------------------------ optimizer step of one adapter
    def _step_adapter(self, adapter: int, num_microbatches: int) -> None:
        arena = self.stage.arena
        if self.layout.tp > 1:
            self.stage.reduce_replicated_grads(adapter)
        scale = 1.0 / (max(num_microbatches, 1) * self.layout.dp)
        if self._fused is not None:
            self._fused.reduce_and_step(adapter, grad_scale=scale)
            return
        if self.layout.dp > 1:
            arena.all_reduce_adapter_grads(adapter, self.state.dp_group)
        o = self.optim
        arena.adam_step(adapter, lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay,
                        grad_scale=scale)

    # ------------------------------------------------------------------ running a schedule
    def shard_tokens(self, tokens: int) -> int:
        return tokens // self.layout.tp

    def prepare(self, provider: MockMultiLoRADataProvider, start: int = 0, stop: Optional[int] = None) -> list:
        """Stage + copy the microbatches ``[start, stop)`` of the provider's schedule."""
        out = []
        for mb in provider.microbatches(start, stop):
            if mb.is_empty:
                out.append(PipelineMicrobatch(None, 0, is_empty=True))
                continue
            batch = provider.to_device(mb, self.device)
            if self.layout.tp > 1 and batch.num_tokens % (128 * self.layout.tp):
                raise ValueError(f"microbatch of {batch.num_tokens} tokens is not divisible by 128 x tp")
            out.append(PipelineMicrobatch(batch, self.shard_tokens(batch.num_tokens)))
        return out

    def run(self, microbatches: Sequence[PipelineMicrobatch]) -> PipelineStats:
        return self.runtime.run(microbatches)
