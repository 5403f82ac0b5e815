"""Multi-GPU multi-LoRA training / benchmarking driver (dp x pp x tp).

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 -m lorafusion_b200.cli.train \
        --model_name_or_path llama-3.1-70b --load_in_4bit true --use_multi_lora true \
        --num_multi_loras 4 --multi_lora_r "16" --pipeline_parallel_size 2 \
        --tensor_parallel_size 4 --multi_lora_max_microbatch_tokens 16384 \
        --multi_lora_global_batch_sizes "8 8 8 8" --max_steps 4

Counterpart of ``benchmarks_paper/bench_multi_gpu.py`` (+ ``scripts/run_single.sh``): parses
the three argument groups, builds the model stage of this rank, obtains a microbatch schedule
(solver or ``--multi_lora_dataset_schedule_path``), runs ``max_steps`` global batches through
1F1B with per-adapter optimizer steps, and reports device-timed throughput (real tokens/s,
summed over data-parallel replicas, max time over ranks), the bubble ratio and peak memory.
Results are appended to ``<output_dir>/results.csv``.  ``--benchmark_baseline_mlora_schedule``
runs the mLoRA-style schedule (no bin packing, one sample of every adapter per microbatch)
through the same runtime for comparison.
"""

from __future__ import annotations

import csv
import json
import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

from ..models.config import get_model_config
from ..ops import _native
from ..simulator import pipeline_sim as ps
from ..solver import schedule as S
from ..train.checkpoint import CheckpointLayout, load_checkpoint, save_checkpoint
from ..train.args import parse_args_into_dataclasses, parse_list
from ..train.engine import EngineConfig, ParallelTrainer
from ..train.provider import MockMultiLoRADataProvider
from ..train.trainer import OptimizerConfig
from ..utils.logging import log_rank0, setup_logging


def main(argv=None) -> dict:
    margs, targs, dargs = parse_args_into_dataclasses(argv)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=device)
    setup_logging(rank)
    health = None
    if world > 1:
        # heartbeats + failure notes in the rendezvous store: a rank that raised or left is
        # noticed before the next launch instead of by a device-side wait running out
        from ..parallel.health import HealthMonitor

        health = HealthMonitor(dist.distributed_c10d._get_default_store(), rank, world, timeout=120.0).start()
    try:
        return _run(margs, targs, dargs, rank, world, device, health)
    except Exception as e:  # noqa: BLE001
        if health is not None:
            health.report_failure(f"{type(e).__name__}: {e}")
        raise
    finally:
        if health is not None:
            health.stop()


def _run(margs, targs, dargs, rank, world, device, health) -> dict:

    cfg = get_model_config(margs.model_name_or_path)
    if margs.num_layers_for_debugging:
        cfg = cfg.with_layers(margs.num_layers_for_debugging)
    adapters = margs.adapter_specs()
    pp, tp = targs.pipeline_parallel_size, targs.tensor_parallel_size
    dp = world // (pp * tp)
    gbs_global = parse_list(targs.multi_lora_global_batch_sizes, int)
    if len(gbs_global) == 1:
        gbs_global = gbs_global * len(adapters)
    gbs_local = [max(1, g // dp) for g in gbs_global]
    engine = EngineConfig(layout=f"dp{dp}pp{pp}tp{tp}", quantize=margs.load_in_4bit,
                          recompute=targs.recompute_mode(), grad_sync=targs.grad_sync,
                          capacity=targs.multi_lora_max_microbatch_tokens, seed=targs.seed, init_b_std=0.01,
                          use_timers=targs.use_timers, use_fsdp=targs.use_fsdp)
    optim = OptimizerConfig(targs.learning_rate, targs.adam_beta1, targs.adam_beta2, targs.adam_epsilon,
                            targs.weight_decay)
    t0 = time.time()
    trainer = ParallelTrainer(cfg, adapters, [g * dp for g in gbs_local], device, engine, optim, health=health)
    log_rank0(f"model {cfg.name} ({engine.layout}) built in {time.time() - t0:.1f}s; "
              f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated")

    ckpt_layout = CheckpointLayout.from_parallel_state(trainer.state, fused_dp=trainer.grad_sync == "fused")
    start_batches, index_offset = None, 0
    if targs.resume_from:
        # adapters (PEFT layout) and optimizer state written by --save_adapters of an earlier run,
        # under any dp x pp x tp layout; the data of every adapter continues where it stopped
        metas = load_checkpoint(trainer.stage.arena, targs.resume_from, ckpt_layout)
        start_batches = [0] * len(adapters)
        for i, (a, meta) in enumerate(zip(adapters, metas)):
            if meta is not None:
                start_batches[i] = int(meta["data_cursor"]) // gbs_global[i]
                index_offset = max(index_offset, int(meta["extra"].get("microbatches", 0)))
                log_rank0(f"resumed {a.name}: optimizer step {meta['step']}, data cursor {meta['data_cursor']}")

    names = parse_list(dargs.adapter_to_dataset, str)
    names = (names * len(adapters))[:len(adapters)]
    provider = MockMultiLoRADataProvider.from_named_distributions(
        adapters, names, gbs_local, num_samples=max(dargs.num_samples, max(gbs_local) * (targs.max_steps + 1 + max(start_batches or [0]))),
        seed=dargs.dataset_seed, max_len=min(dargs.max_seq_len, engine.capacity), capacity=engine.capacity,
        num_pipeline_stages=pp, vocab_size=cfg.vocab_size, schedule_path=dargs.multi_lora_dataset_schedule_path,
        num_global_batches=targs.max_steps, dp_rank=trainer.state.dp_rank, total_multiple=128 * tp,
        start_global_batches=start_batches, index_offset=index_offset)
    if targs.benchmark_baseline_mlora_schedule:
        sched = ps.generate_mlora_schedule(provider.data, engine.capacity)
        _, _, sched = S.verify_correctness_of_schedule(provider.data, sched, pp, add_bubble=True)
        provider.schedule, provider.flat = sched, S.flatten_schedule(sched)
    log_rank0(f"schedule: {json.dumps(provider.statistics())}")

    mbs = trainer.prepare(provider)
    if health is not None:
        health.check()
    n_warm = min(len(mbs) // 4, 2 * pp)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if n_warm:
        # warm-up on a copy of the first microbatches with the optimizer hooks disabled
        saved_mgr = trainer.runtime.manager
        trainer.runtime.manager = None
        trainer.run(mbs[:n_warm])
        trainer.stage.arena.zero_grad()
        trainer.runtime.manager = saved_mgr
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if health is not None:
        health.check()
    torch.cuda.reset_peak_memory_stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    from ..utils.benchmark import create_profiler_context

    e0.record()
    with create_profiler_context(enabled=targs.profile and rank == 0,
                                 output_dir=str(Path(targs.output_dir) / "profile"), scheduled=False):
        stats = trainer.run(mbs)
    e1.record()
    torch.cuda.synchronize()
    _native.check_device_errors()
    ms = e0.elapsed_time(e1)
    tokens = sum(m.info.total_tokens for m in provider.microbatches())
    agg = torch.tensor([ms, float(tokens) if trainer.state.pp_rank == 0 and trainer.state.tp_rank == 0 else 0.0,
                        torch.cuda.max_memory_allocated() / 2**30], dtype=torch.float64, device=device)
    if world > 1:
        mx = agg.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = agg.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, tokens, peak = float(mx[0]), float(sm[1]), float(mx[2])
    else:
        peak = float(agg[2])
    result = {
        "model": cfg.name, "layout": engine.layout, "world": world, "adapters": len(adapters),
        "capacity": engine.capacity, "microbatches": len(mbs), "tokens": tokens, "time_ms": ms,
        "throughput_tokens_per_s": tokens / (ms / 1e3), "throughput_per_gpu": tokens / (ms / 1e3) / world,
        "peak_memory_gib": peak, "bubble_ratio": stats.bubble_ratio if targs.use_timers else None,
        "optimizer_steps": trainer.manager.steps_taken, "quantized": margs.load_in_4bit,
        "schedule": "mlora" if targs.benchmark_baseline_mlora_schedule else "solver",
    }
    if rank == 0:
        out = Path(targs.output_dir)
        out.mkdir(parents=True, exist_ok=True)
        new = not (out / "results.csv").exists()
        with open(out / "results.csv", "a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(result))
            if new:
                w.writeheader()
            w.writerow(result)
        print(json.dumps(result))
    if targs.save_adapters:
        save_checkpoint(trainer.stage.arena, targs.output_dir, ckpt_layout, base_model_name=cfg.name,
                        data_cursors=[((start_batches or [0] * len(adapters))[i] + trainer.manager.steps_taken.get(i, 0))
                                      * gbs_global[i] for i in range(len(adapters))],
                        extra={"microbatches": index_offset + len(mbs)})
    if world > 1:
        dist.barrier()
        if health is not None:
            health.stop()
        dist.destroy_process_group()
    return result


if __name__ == "__main__":
    main(sys.argv[1:])
