"""Benchmark of the fused compute + collective kernels against their unfused NCCL baselines,
with the achieved fraction of each path's roofline.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 -m lorafusion_b200.cli.bench_collectives \
        --model llama-3.1-70b --tokens 16384

For the tensor-parallel shapes of ``--model`` at TP = world size it times, device-side and as the
maximum over ranks:

* all-gather -> GEMM   (column-parallel qkv and gate|up): the fused kernel (``tp_ops.ag_gemm``)
  vs ``all_gather_into_tensor`` + the plain tcgen05 GEMM;
* GEMM -> reduce-scatter (row-parallel o and down): the fused kernel (``tp_ops.gemm_rs``) vs the
  plain GEMM + ``reduce_scatter_tensor``;
* LoRA gradient reduce-scatter + AdamW + all-gather (data parallel over the same ranks): the fused
  kernel (``dp_sync.FusedGradSync``) vs NCCL all-reduce + the local Adam kernel.

Roofline of a fused path = the slower of (FLOPs / measured bf16 GEMM peak) and (bytes that must
cross NVLink per GPU / measured per-direction link bandwidth); the fraction reported is that
time divided by the measured time.  With one rank the peers are this GPU itself (loop-back), which
measures the overhead of the communication warps and flags on top of the plain GEMM.
The reference performs these steps as separate Megatron / NCCL calls without overlap
(``lorafusion/ops/multi_lora.py:166-184``, ``benchmarks_paper/bench_multi_gpu.py:135-149``).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..models.adapters import LoRAArena
from ..models.config import AdapterSpec, get_model_config
from ..ops import _native
from ..ops.gemm import gemm_nt
from ..parallel.dp_sync import FusedGradSync, NcclGradSync
from ..parallel.symmetric import SymmetricAllocator
from ..parallel.tp_ops import TpContext, ag_gemm, gemm_rs
from ..train.trainer import OptimizerConfig

GEMM_PEAK_TFLOPS = 1375.8   # measured sustained cuBLAS bf16 on this pool's B200
LINK_GBS = 770.0            # measured peer copy bandwidth per direction per GPU


def _time(fn, device, world, warmup: int, number: int) -> float:
    """Seconds per call: CUDA events on the launching stream, barrier + synchronize around the
    timed region, maximum over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(number):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    t = torch.tensor([e0.elapsed_time(e1) / number / 1e3], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run(args) -> list:
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=device)
    group = dist.group.WORLD if world > 1 else None
    cfg = get_model_config(args.model)
    T, H, I = args.tokens, cfg.hidden_size, cfg.intermediate_size
    if T % (128 * world):
        raise SystemExit("--tokens must be a multiple of 128 x world size")
    ms = T // world
    torch.manual_seed(rank)
    results = []

    def emit(row):
        results.append(row)
        if rank == 0:
            print(json.dumps(row))

    ctx = TpContext(group, device, max_tokens=T, max_features=max(H, cfg.qkv_size // world, 2 * I // world))
    kw = dict(device=device, world=world, warmup=args.warmup, number=args.number)

    # ---------------- all-gather -> GEMM (column parallel) ----------------
    for name, n_full in (() if args.only_dp else (("qkv", cfg.qkv_size), ("gate_up", 2 * I))):
        n_loc = n_full // world
        w = (torch.randn(n_loc, H, device=device) * 0.02).to(torch.bfloat16)
        x_loc = torch.randn(ms, H, device=device).to(torch.bfloat16)
        ctx.own_gather_rows(T, H).copy_(x_loc)
        out = torch.empty(T, n_loc, dtype=torch.bfloat16, device=device)
        gathered = torch.empty(T, H, dtype=torch.bfloat16, device=device)

        def fused():
            ag_gemm(ctx, T, H, w, out=out)

        def unfused():
            if world > 1:
                dist.all_gather_into_tensor(gathered, x_loc, group=group)
            else:
                gathered.copy_(x_loc)
            gemm_nt(gathered, w, out=out)

        t_f, t_u = _time(fused, **kw), _time(unfused, **kw)
        flops = 2.0 * T * H * n_loc
        link_bytes = (world - 1) * ms * H * 2  # what each GPU must receive (and send)
        roof = max(flops / (GEMM_PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9))
        emit({"path": f"all-gather->GEMM {name}", "world": world, "shape": f"[{T} x {H}] x [{n_loc} x {H}]^T",
              "fused_ms": t_f * 1e3, "nccl_plus_gemm_ms": t_u * 1e3, "speedup": t_u / t_f,
              "tflops": flops / t_f / 1e12, "roofline_ms": roof * 1e3, "roofline_fraction": roof / t_f,
              "bound": "compute" if flops / (GEMM_PEAK_TFLOPS * 1e12) >= link_bytes / (LINK_GBS * 1e9) else "link"})
        del w, out, gathered

    # ---------------- GEMM -> reduce-scatter (row parallel) ----------------
    for name, k_full in (() if args.only_dp else (("o", cfg.q_size), ("down", I))):
        k_loc = k_full // world
        w = (torch.randn(H, k_loc, device=device) * 0.02).to(torch.bfloat16)
        x = torch.randn(T, k_loc, device=device).to(torch.bfloat16)
        out = torch.empty(ms, H, dtype=torch.bfloat16, device=device)
        partial = torch.empty(T, H, dtype=torch.bfloat16, device=device)

        def fused():
            gemm_rs(ctx, x, w, out=out)

        def unfused():
            gemm_nt(x, w, out=partial)
            if world > 1:
                dist.reduce_scatter_tensor(out, partial, group=group)
            else:
                out.copy_(partial[:ms])

        t_f, t_u = _time(fused, **kw), _time(unfused, **kw)
        flops = 2.0 * T * k_loc * H
        link_bytes = (world - 1) * ms * H * 2
        roof = max(flops / (GEMM_PEAK_TFLOPS * 1e12), link_bytes / (LINK_GBS * 1e9))
        emit({"path": f"GEMM->reduce-scatter {name}", "world": world, "shape": f"[{T} x {k_loc}] x [{H} x {k_loc}]^T",
              "fused_ms": t_f * 1e3, "gemm_plus_nccl_ms": t_u * 1e3, "speedup": t_u / t_f,
              "tflops": flops / t_f / 1e12, "roofline_ms": roof * 1e3, "roofline_fraction": roof / t_f,
              "bound": "compute" if flops / (GEMM_PEAK_TFLOPS * 1e12) >= link_bytes / (LINK_GBS * 1e9) else "link"})
        del w, x, out, partial
    del ctx
    torch.cuda.empty_cache()

    # ---------------- LoRA gradient sync + AdamW (data parallel) ----------------
    layers = args.dp_layers
    adapters = [AdapterSpec(f"lora_{i}", r=16) for i in range(4)]
    optim = OptimizerConfig(lr=1e-4)
    alloc = SymmetricAllocator(device, group) if world > 1 else None
    arena_f = LoRAArena(cfg, adapters, range(layers), device, init_b_std=0.01, shared_alloc=alloc)
    arena_n = LoRAArena(cfg, adapters, range(layers), device, init_b_std=0.01)
    nccl = NcclGradSync(arena_n, group, optim)
    if world > 1:
        fused_sync = FusedGradSync(arena_f, alloc, group, optim)

        def fused():
            for a in range(len(adapters)):
                fused_sync.reduce_and_step(a, grad_scale=1.0 / world)
    else:
        def fused():
            for a in range(len(adapters)):
                arena_f.adam_step(a, lr=optim.lr, grad_scale=1.0)

    def unfused():
        if world > 1:
            nccl.all_reduce()
        for a in range(len(adapters)):
            nccl.reduce_and_step(a, grad_scale=1.0 / world)

    t_f, t_u = _time(fused, **kw), _time(unfused, **kw)
    extra = {}
    if world > 1:
        # where the fused kernel's time goes, from its own time stamps (one launch, adapter 0)
        from ..parallel.dp_sync import summarize_sync_trace

        fused_sync.trace = torch.zeros(3 * 65536, dtype=torch.int64, device=device)
        fused_sync.reduce_and_step(0, grad_scale=1.0 / world)
        torch.cuda.synchronize()
        tr = summarize_sync_trace(fused_sync.trace, fused_sync.last_num_items)
        extra["in_kernel_us"] = {k: round(v, 1) for k, v in tr.items() if k.endswith("_us")}
        fused_sync.trace = None
    if world > 1 and args.multimem:
        # same kernel with NVLS: multimem.ld_reduce pulls the sum of all ranks' gradients through the
        # switch, multimem.st broadcasts the new weights
        arena_m = LoRAArena(cfg, adapters, range(layers), device, init_b_std=0.01, shared_alloc=alloc)
        mm_sync = FusedGradSync(arena_m, alloc, group, optim, use_multimem=True)
        if mm_sync.use_multimem:
            def fused_mm():
                for a in range(len(adapters)):
                    mm_sync.reduce_and_step(a, grad_scale=1.0 / world)

            extra["fused_multimem_ms"] = _time(fused_mm, **kw) * 1e3
        else:
            extra["fused_multimem_ms"] = None
            extra["multimem_note"] = "no multicast address for the symmetric buffers on this system"
    n_pad = arena_f.numel
    n_train = sum(arena_f.trainable_numel(a) for a in range(len(adapters)))
    # per GPU: receive (world-1)/world of the fp32 gradients, send the same share of bf16 weights to each peer
    link_bytes = (world - 1) / world * n_pad * 4 if world > 1 else 0.0
    hbm_bytes = n_pad * 4 * 2 + n_train * (3 * 8 + 2)  # read + clear gradients, state read/write, bf16 weights
    roof = max(link_bytes / (LINK_GBS * 1e9), hbm_bytes / 6546e9 / max(world, 1))
    emit({"path": "LoRA grad reduce-scatter + AdamW + all-gather", "world": world,
          "shape": f"{layers} layers x 4 adapters r16: {n_pad / 1e6:.0f}M padded / {n_train / 1e6:.0f}M trainable elements",
          "fused_ms": t_f * 1e3, "nccl_allreduce_plus_adam_ms": t_u * 1e3, "speedup": t_u / t_f,
          "roofline_ms": roof * 1e3, "roofline_fraction": roof / t_f, **extra,
          "bound": "link" if link_bytes / (LINK_GBS * 1e9) >= hbm_bytes / 6546e9 / max(world, 1) else "hbm"})
    _native.check_device_errors()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return results


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="llama-3.1-70b")
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--dp-layers", type=int, default=8, help="layers of adapters in the gradient-sync case")
    ap.add_argument("--multimem", action="store_true",
                    help="also time the gradient-sync kernel on its NVLS path (multimem.ld_reduce / multimem.st)")
    ap.add_argument("--only-dp", action="store_true", help="skip the tensor-parallel cases")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--number", type=int, default=10)
    run(ap.parse_args(argv))


if __name__ == "__main__":
    main()
