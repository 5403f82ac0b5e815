"""Headline benchmark: training tokens/s of multi-LoRA fine-tuning on a Llama-3.1-70B-shaped
decoder (NF4 frozen base, 4 LoRA adapters of rank 16 on all linears, mixed sequence-length
distributions, 16K-token packed microbatches) on N B200s of one node.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One *step* = every rank runs forward + backward of ``--microbatches`` packed microbatches
(all four adapters batched together in each), the LoRA gradients are reduced over the
data-parallel group, and every adapter takes an AdamW step.  Weak scaling: per-GPU work is
fixed as N grows.  Throughput counts real (unpadded) tokens summed over all GPUs.

Two measurements come out of ONE pass over the K timed steps (CUDA events, max over ranks):
* ``e2e``    -- the whole pass: every step copies its token arrays from pinned host memory to
  the device, computes, and reads the loss back to the host;
* ``value``  -- the compute part alone (forward, backward, gradient reduction, optimizer), summed
  over the steps.

Every step's microbatches are packed by the solver from one pool of samples for the whole
data-parallel group and dealt so that all ranks get the same number of nearly full microbatches
and about the same attention work (``train.data.pack_balanced_dp_step``).

``--impl reference`` reports why the reference itself cannot be run here.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

# Grow allocator segments in place: with fixed-size segments a third of a B200 ends up as
# cached-but-unusable fragments next to the multi-GB activation tensors of a 70B layer.
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

H100_PER_GPU_TOKENS_PER_S = 5115.41 / 4  # reference LoRAFusion, 70B mixed, 4xH100 (published)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3.1-70b")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debug only)")
    ap.add_argument("--capacity", type=int, default=16384, help="tokens per microbatch")
    ap.add_argument("--microbatches", type=int, default=2, help="microbatches per step per GPU")
    ap.add_argument("--dropout", type=float, default=0.1)
    ap.add_argument("--no-quantize", action="store_true")
    ap.add_argument("--recompute", default="auto", choices=["auto", "all", "none"],
                    help="activation recomputation: all layers, none, or as memory allows")
    ap.add_argument("--skip-e2e", action="store_true", help="accepted for compatibility; both numbers come from one pass")
    ap.add_argument("--offload", default="auto", choices=["auto", "on", "off"],
                    help="park gate|up activations in pinned host memory over PCIe; auto = time one step "
                         "with and without during set-up and keep the faster plan")
    ap.add_argument("--grad-sync", default="auto", choices=["auto", "fused", "nccl"],
                    help="DP gradient path: fused reduce+Adam kernel over peer memory, or NCCL all-reduce")
    ap.add_argument("--lora-mode", default="fused", choices=["fused", "unfused"],
                    help="unfused = same-GPU baseline: separate base GEMM + cuBLAS LoRA GEMMs + stored mask")
    ap.add_argument("--multimem", action="store_true", help="use NVLS multimem loads/stores in the fused sync")
    ap.add_argument("--layout", default="auto", choices=["auto", "dp", "tp2"],
                    help="dp = one replica per GPU; tp2 = every pair of GPUs shares a replica (tensor + sequence "
                         "parallel, fused all-gather->GEMM / GEMM->reduce-scatter kernels), data parallel over "
                         "the pairs; auto = tp2 on an even number of GPUs, where halving every kept activation "
                         "removes the recomputation a 70B replica needs on one GPU")
    ap.add_argument("--fsdp", action="store_true",
                    help="baseline: base weights sharded over the GPUs and all-gathered per layer (ZeRO-3 style)")
    ap.add_argument("--seed", type=int, default=1234, help="seed of the synthetic sample lengths")
    return ap.parse_args()


def reference_arm(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:   # one line per job, from rank 0
        return
    print(json.dumps({
        "impl": "reference",
        "unavailable": "pip install of the reference yields only lorafusion/__init__.py (its pyproject lists "
                       "packages=['lorafusion'] without sub-packages) and its training path needs "
                       "megatron.core, peft, trl and bitsandbytes, none of which is installed; its TMA "
                       "kernels use Triton-3.2-only APIs absent from the installed Triton 3.6",
    }))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_all_step_specs(seed: int, capacity: int, per_rank: int, world: int, n_steps: int):
    """``specs[step][rank]`` = the microbatches of every rank for every step.  Samples are drawn
    round-robin from the four adapters' length distributions (lognormal medians
    256/512/1024/2048, sigma 0.5-0.8, clipped to [32, 8192]) into a pool a little larger than
    the step needs; the solver packs it, and what it leaves over opens the next step's pool."""
    import numpy as np

    from lorafusion_b200.train.data import LengthDistribution, pack_balanced_dp_step

    dists = [LengthDistribution(256, 0.5, 32, 8192), LengthDistribution(512, 0.6, 32, 8192),
             LengthDistribution(1024, 0.7, 32, 8192), LengthDistribution(2048, 0.8, 32, 8192)]
    rng = np.random.default_rng(seed)
    out, pool, a = [], [], 0
    for _ in range(n_steps):
        while sum(n for _, n in pool) < world * per_rank * capacity * 1.08:
            pool.append((a, int(dists[a].sample(1, int(rng.integers(1 << 31)))[0])))
            a = (a + 1) % 4
        dealt, pool = pack_balanced_dp_step(pool, world, per_rank, capacity)
        out.append(dealt)
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)

    from lorafusion_b200.models.config import AdapterSpec, get_model_config
    from lorafusion_b200.ops import _native
    from lorafusion_b200.train.data import h2d_bytes
    from lorafusion_b200.train.trainer import MultiLoRATrainer, OptimizerConfig

    if args.lora_mode == "unfused":
        from lorafusion_b200.ops.lora import set_unfused_baseline

        set_unfused_baseline(True)
    cfg = get_model_config(args.model)
    if args.layers > 0:
        cfg = cfg.with_layers(args.layers)
    adapters = [AdapterSpec(f"lora_{i}", r=16, lora_alpha=32.0, dropout=args.dropout) for i in range(4)]
    tp = 2 if (args.layout == "tp2" or (args.layout == "auto" and world >= 2 and world % 2 == 0 and not args.fsdp
                                        and args.lora_mode == "fused" and args.grad_sync != "nccl")) else 1
    if world % tp:
        raise SystemExit(f"--layout tp2 needs an even number of GPUs, got {world}")
    dp = world // tp
    dp_group = tp_group = None
    dp_rank, tp_rank = rank, 0
    if world > 1:
        from lorafusion_b200.parallel.layout import ParallelLayout, initialize_parallel_state

        state = initialize_parallel_state(ParallelLayout(world, dp=dp, pp=1, tp=tp))
        dp_group, tp_group, dp_rank, tp_rank = state.dp_group, state.tp_group, state.dp_rank, state.tp_rank
    per_replica = args.microbatches * tp   # microbatches a replica (one GPU, or one tp pair) runs per step
    t0 = time.time()
    trainer = MultiLoRATrainer(cfg, adapters, device, quantize=not args.no_quantize,
                               recompute={'auto': 'auto', 'all': True, 'none': False}[args.recompute], optim=OptimizerConfig(lr=1e-4),
                               dp_group=dp_group if dp > 1 else None, seed=1234, init_b_std=0.01,
                               grad_sync=args.grad_sync, use_multimem=args.multimem, use_fsdp=args.fsdp,
                               tp_group=tp_group if tp > 1 else None, max_tokens=args.capacity)
    if "expandable_segments:True" in os.environ.get("PYTORCH_CUDA_ALLOC_CONF", ""):
        trainer.stage.reserve_bytes = 5 << 30  # little fragmentation to provide for
    trainer.stage.plan_activations(args.capacity)
    torch.cuda.synchronize()
    if rank == 0:
        print(f"[bench] model {cfg.name} built in {time.time() - t0:.1f}s, base weights "
              f"{trainer.stage.base_weight_bytes() / 2**30:.1f} GiB, device mem "
              f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB", file=sys.stderr)

    n_total = args.warmup + args.steps
    # Rank 0 packs every step for the whole group (the branch and bound stops on a time limit,
    # so two ranks could find different packings) and hands every rank its share.
    box = [make_all_step_specs(args.seed, args.capacity, per_replica, dp, n_total + 1)
           if rank == 0 else None]
    if world > 1:
        dist.broadcast_object_list(box, src=0)
    all_specs = box[0]
    for st_ in all_specs:
        for per in st_:
            for sp in per:
                sp.total_multiple = 128 * tp   # token rows are cut in tp equal shards of whole tiles
    step_specs = [all_specs[s][dp_rank] for s in range(n_total)]   # both ranks of a tp pair run the same batches
    probe_specs = all_specs[n_total][dp_rank]
    tokens_per_step = [sum(sp.total_tokens for sp in specs) for specs in step_specs]
    sq = [sum(n * n for sp in st_[r] for _, lens in sp.segments for n in lens) for st_ in all_specs[:n_total]
          for r in range(dp)]
    balance = {"attention_cost_max_over_mean": round(max(
        max(sq[s * dp:(s + 1) * dp]) * dp / max(sum(sq[s * dp:(s + 1) * dp]), 1)
        for s in range(n_total)), 3)}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def agree(flag: bool) -> bool:
        """True only if every rank says True."""
        t = torch.tensor([1.0 if flag else 0.0], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() > 0.5)

    def timed_step(batches) -> float:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        trainer.step_on_device(batches)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- set-up (untimed): choose the activation plan by measurement ----
    # One warm step and one timed step without offloading; then, if the host link measured
    # under the load of all ranks can take at least a few layers per forward pass, one timed
    # step with that many layers' gate|up parked in host memory.  The faster plan stays.
    offload_note, like_for_like = "off", None
    host0 = trainer.stage_batches(probe_specs, n_total)
    dev0 = trainer.to_device(probe_specs, host0, n_total)
    probe_tokens = sum(sp.total_tokens for sp in probe_specs)
    trainer.step_on_device(dev0)
    t_off = 0.0
    if tp == 1:
        t_off = timed_step(dev0)
        like_for_like = {"policy": "data parallel, no host offload",
                         "ms_per_step": round(t_off, 1), "tokens_per_s_per_gpu": round(probe_tokens / (t_off / 1e3), 1),
                         "steps": 1}
    else:
        offload_note = "off (not needed: a tp2 replica keeps every layer's activations on its two GPUs)"
    if tp == 1 and args.offload != "off" and args.recompute == "auto" and args.lora_mode == "fused":
        from lorafusion_b200.models.offload import measure_pcie_bandwidth

        d2h, h2d = measure_pcie_bandwidth(device, dist.group.WORLD if world > 1 else None)
        # (all GPUs of the node copy at once, whatever group they belong to)
        per_gu = args.capacity * 2 * cfg.intermediate_size * 2
        fwd_s = (t_off / 1e3) / args.microbatches / 3.0   # a forward pass is about a third of fwd + bwd
        # the forward pass sends, the (twice as long) backward pass fetches
        n_link = int(0.9 * min(d2h * fwd_s, h2d * 2.0 * fwd_s) / per_gu)
        offload_note = f"off (host link {d2h / 1e9:.1f} / {h2d / 1e9:.1f} GB/s out / in takes {n_link} layers per forward pass)"
        if (n_link >= 6 or args.offload == "on") and agree(trainer.stage.prepare_offload(args.capacity, max_layers=n_link)):
            t_on = timed_step(dev0)
            n_off = trainer.stage.keep_summary(args.capacity)["gate_up_in_host_memory"]
            waits = trainer.stage._offloader.backlog_waits
            detail = (f"{n_off} layers, host link {d2h / 1e9:.1f} / {h2d / 1e9:.1f} GB/s out / in under the load of "
                      f"all ranks, set-up step {t_on:.0f} ms vs {t_off:.0f} ms without, {waits} backlog waits")
            if args.offload == "on" or t_on < 0.995 * t_off:
                offload_note = "on, " + detail
            else:
                offload_note = "off (tried " + detail + ")"
                trainer.stage.disable_offload()
                torch.cuda.empty_cache()
        elif trainer.stage.offload_enabled:
            trainer.stage.disable_offload()
    del dev0, host0

    # ---- the timed pass: warm-up steps, then K steps end to end ----
    host = [trainer.stage_batches(specs, s) for s, specs in enumerate(step_specs)]
    last_loss = float("nan")
    for s in range(args.warmup):
        last_loss = trainer.train_step(step_specs[s], s, host=host[s])
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _native.launch_count()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.steps)]
    ev_begin, ev_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    bytes_in = 0
    ev_begin.record()
    for k, s in enumerate(range(args.warmup, n_total)):
        batches = trainer.to_device(step_specs[s], host[s], s)     # host -> device, from pinned memory
        ev[k][0].record()
        loss_dev = trainer.step_on_device(batches)
        ev[k][1].record()
        last_loss = float(loss_dev.item())                          # device -> host, 4 bytes
        if k == 0:
            bytes_in = sum(h2d_bytes(b) for b in batches)
        del batches
    ev_end.record()
    barrier()
    clocks = sampler.stop()
    launches = _native.launch_count() - launches0
    ms_e2e = ev_begin.elapsed_time(ev_end)
    step_ms = [a.elapsed_time(b) for a, b in ev]
    ms = sum(step_ms)
    toks = float(sum(tokens_per_step[args.warmup:])) if tp_rank == 0 else 0.0   # a tp pair's tokens count once
    stats = torch.tensor([ms, ms_e2e, toks], dtype=torch.float64, device=device)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, ms_e2e, toks = float(mx[0]), float(mx[1]), float(sm[2])
        per_step = torch.tensor(step_ms, dtype=torch.float64, device=device)
        dist.all_reduce(per_step, op=dist.ReduceOp.MAX)
        step_ms = per_step.tolist()
    _native.check_device_errors()
    loss_val = last_loss
    value = toks / (ms / 1e3)
    result = {
        "metric": "training tokens/s, multi-LoRA Llama-3.1-70B, 1/2/4/8 B200, max over ranks",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": value / (H100_PER_GPU_TOKENS_PER_S * world),
        "dtype": "bf16",
        "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": cfg.name + ("-nf4" if not args.no_quantize else "-bf16"),
            "global_batch": f"{args.microbatches} x {args.capacity}-token microbatches per GPU per step"
                            + (f" ({per_replica} per tp{tp} replica)" if tp > 1 else ""),
            "seq_len": "lognormal medians 256/512/1024/2048, sigma 0.5-0.8, clip [32,8192], packed",
            "parallelism": (f"dp{dp}tp{tp}" if tp > 1 else f"dp{world}")
                           + (" + base sharded ZeRO-3 style (baseline)" if args.fsdp else ""),
            "adapters": "4 x LoRA r16 alpha32 dropout %.2f on q,k,v,o,gate,up,down" % args.dropout,
            "grad_sync": trainer.grad_sync,
            "lora_mode": args.lora_mode,
            "recompute": args.recompute,
            "layers_without_recompute": trainer.stage.keep_summary(args.capacity)["keep_all_gemm_outputs"],
            "activation_plan": trainer.stage.keep_summary(args.capacity),
            "activation_offload": offload_note,
            "l2": "inputs (frozen base weights) far larger than L2",
            "baseline": "vs_baseline = value / (n_gpus * 1278.85 tok/s/GPU), the reference's published "
                        "70B-mixed LoRAFusion throughput on 4xH100 per GPU",
            "tokens_per_step_per_gpu": tokens_per_step[-1] // tp,
            "batches": "solver-packed per step for the whole dp group, dealt by sum(len^2) "
                       "(train.data.pack_balanced_dp_step)",
            "balance": balance,
            "same_policy_at_every_n": like_for_like,
            "step_ms_max_over_ranks": [round(v, 3) for v in step_ms],
            "final_loss": loss_val,
            "peak_memory_gib": {"allocated": round(torch.cuda.max_memory_allocated() / 2**30, 1),
                                "reserved": round(torch.cuda.max_memory_reserved() / 2**30, 1)},
        },
        "clocks": clocks,
        "gpu_launches": launches,
    }
    result["e2e"] = {
        "value": toks / (ms_e2e / 1e3),
        "unit": "tokens/s",
        "h2d_bytes_per_step": bytes_in,
        "d2h_bytes_per_step": 4,
        "ms_per_step": ms_e2e / args.steps,
        "note": "same K steps as value: one event pair around the whole pass (host-to-device copy of every "
                "step's token arrays from pinned memory, compute, loss read back to the host every step); "
                "value sums the compute intervals inside it",
    }
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
