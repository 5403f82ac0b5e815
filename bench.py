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

Two measurements are reported:
* ``value``  -- device-timed (CUDA events, max over ranks) with the step's batches already
  resident on the GPU;
* ``e2e``    -- the same K steps through ``MultiLoRATrainer.train_step``: token arrays start
  in pinned host memory and are copied host-to-device every step, and the loss is read back
  to the host every step.

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
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--offload", default="auto", choices=["auto", "on", "off"],
                    help="park gate|up activations in pinned host memory over PCIe; auto = time one step "
                         "with and without during set-up and keep the faster plan")
    ap.add_argument("--grad-sync", default="auto", choices=["auto", "fused", "nccl"],
                    help="DP gradient path: fused reduce+Adam kernel over peer memory, or NCCL all-reduce")
    ap.add_argument("--lora-mode", default="fused", choices=["fused", "unfused"],
                    help="unfused = same-GPU baseline: separate base GEMM + cuBLAS LoRA GEMMs + stored mask")
    ap.add_argument("--multimem", action="store_true", help="use NVLS multimem loads/stores in the fused sync")
    return ap.parse_args()


def reference_arm(args) -> None:
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


def make_step_specs(rng_seed: int, capacity: int, n_microbatches: int):
    """Microbatches of one step: samples are drawn round-robin from the four adapters' length
    distributions (lognormal medians 256/512/1024/2048, sigma 0.5-0.8, clipped to [32, 8192])
    until a microbatch's padded token count would exceed the capacity."""
    import numpy as np

    from lorafusion_b200.train.data import LengthDistribution, MicroBatchSpec

    dists = [LengthDistribution(256, 0.5, 32, 8192), LengthDistribution(512, 0.6, 32, 8192),
             LengthDistribution(1024, 0.7, 32, 8192), LengthDistribution(2048, 0.8, 32, 8192)]
    rng = np.random.default_rng(rng_seed)
    specs = []
    for _ in range(n_microbatches):
        per = {a: [] for a in range(4)}

        def padded(p):
            return sum(((sum(v) + 127) // 128) * 128 for v in p.values() if v)

        a, misses = 0, 0
        while misses < 8:
            n = int(dists[a].sample(1, int(rng.integers(1 << 31)))[0])
            per[a].append(n)
            if padded(per) > capacity:
                per[a].pop()
                misses += 1
            a = (a + 1) % 4
        specs.append(MicroBatchSpec([(k, v) for k, v in per.items() if v]))
    return specs


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
    t0 = time.time()
    trainer = MultiLoRATrainer(cfg, adapters, device, quantize=not args.no_quantize,
                               recompute={'auto': 'auto', 'all': True, 'none': False}[args.recompute], optim=OptimizerConfig(lr=1e-4),
                               dp_group=dist.group.WORLD if world > 1 else None, seed=1234, init_b_std=0.01,
                               grad_sync=args.grad_sync, use_multimem=args.multimem)
    if "expandable_segments:True" in os.environ.get("PYTORCH_CUDA_ALLOC_CONF", ""):
        trainer.stage.reserve_bytes = 16 << 30  # little fragmentation to provide for
    trainer.stage.plan_activations(args.capacity)
    torch.cuda.synchronize()
    if rank == 0:
        print(f"[bench] model {cfg.name} built in {time.time() - t0:.1f}s, base weights "
              f"{trainer.stage.base_weight_bytes() / 2**30:.1f} GiB, device mem "
              f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB", file=sys.stderr)

    n_total = args.warmup + args.steps
    step_specs = [make_step_specs(1000 * rank + s, args.capacity, args.microbatches) for s in range(n_total)]
    tokens_per_step = [sum(sp.total_tokens for sp in specs) for specs in step_specs]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run_pass(e2e: bool):
        """Returns (elapsed ms for the timed steps (max over ranks), tokens, clocks, launches)."""
        host = [trainer.stage_batches(specs, s) for s, specs in enumerate(step_specs)]
        dev = None
        if not e2e:
            dev = [trainer.to_device(specs, h, s) for s, (specs, h) in enumerate(zip(step_specs, host))]
        last_loss = None
        for s in range(args.warmup):
            if e2e:
                last_loss = trainer.train_step(step_specs[s], s, host=host[s])
            else:
                trainer.step_on_device(dev[s])
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        launches0 = _native.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for s in range(args.warmup, n_total):
            if e2e:
                last_loss = trainer.train_step(step_specs[s], s, host=host[s])
            else:
                last_loss = trainer.step_on_device(dev[s])
        ev1.record()
        barrier()
        clocks = sampler.stop()
        ms = ev0.elapsed_time(ev1)
        launches = _native.launch_count() - launches0
        toks = sum(tokens_per_step[args.warmup:])
        stats = torch.tensor([ms, float(toks)], dtype=torch.float64, device=device)
        if world > 1:
            mx = stats.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            sm = stats.clone()
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            ms, toks = float(mx[0]), float(sm[1])
        _native.check_device_errors()
        loss_val = float(last_loss) if last_loss is not None else float("nan")
        bytes_in = sum(h2d_bytes(b) for b in (dev[-1] if dev else trainer.to_device(step_specs[-1], host[-1], 0)))
        return ms, toks, clocks, launches, loss_val, bytes_in

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
    offload_note = "off"
    if args.offload != "off" and args.recompute == "auto" and args.lora_mode == "fused":
        host0 = trainer.stage_batches(step_specs[0], 0)
        dev0 = trainer.to_device(step_specs[0], host0, 0)
        trainer.step_on_device(dev0)
        t_off = timed_step(dev0)
        ok = agree(trainer.stage.prepare_offload(args.capacity))
        if ok:
            trainer.step_on_device(dev0)
            t_on = timed_step(dev0)
            n_off = trainer.stage.keep_summary(args.capacity)["gate_up_in_host_memory"]
            waits = trainer.stage._offloader.backlog_waits
            offload_note = f"on, {n_off} layers (set-up step {t_on:.0f} ms vs {t_off:.0f} ms without, {waits} backlog waits)"
            if args.offload == "auto" and not t_on < 0.99 * t_off:
                ok = False
                offload_note = f"off (set-up step {t_on:.0f} ms with {n_off} layers parked vs {t_off:.0f} ms without, {waits} backlog waits)"
        if not ok:
            trainer.stage.disable_offload()
            torch.cuda.empty_cache()
        del dev0, host0

    ms, toks, clocks, launches, loss_val, bytes_in = run_pass(e2e=False)
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
            "global_batch": f"{args.microbatches} x {args.capacity}-token microbatches per GPU per step",
            "seq_len": "lognormal medians 256/512/1024/2048, sigma 0.5-0.8, clip [32,8192], packed",
            "parallelism": f"dp{world}",
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
            "tokens_per_step_per_gpu": tokens_per_step[-1],
            "final_loss": loss_val,
            "peak_memory_gib": {"allocated": round(torch.cuda.max_memory_allocated() / 2**30, 1),
                                "reserved": round(torch.cuda.max_memory_reserved() / 2**30, 1)},
        },
        "clocks": clocks,
        "gpu_launches": launches,
    }
    if not args.skip_e2e:
        ms2, toks2, clocks2, launches2, loss2, bytes_in2 = run_pass(e2e=True)
        result["e2e"] = {
            "value": toks2 / (ms2 / 1e3),
            "unit": "tokens/s",
            "h2d_bytes_per_step": bytes_in2,
            "d2h_bytes_per_step": 4,
            "ms_per_step": ms2 / args.steps,
            "clocks": clocks2,
            "final_loss": loss2,
        }
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
