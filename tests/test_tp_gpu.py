"""Tensor-parallel fused kernels (all-gather -> GEMM, GEMM -> reduce-scatter) on 2 real GPUs,
checked against NCCL collectives + fp32 matmul.  Child processes, NVLS off, plain peer
loads/stores in the kernels."""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

_CHILD = r"""
import os, torch, torch.distributed as dist
os.environ["NCCL_NVLS_ENABLE"] = "0"
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from lorafusion_b200.parallel.tp_ops import TpContext, ag_gemm, gemm_rs
from lorafusion_b200.ops import _native
from lorafusion_b200.utils.testing import assert_close_two_rounds
torch.backends.cuda.matmul.allow_tf32 = False

T_MAX, K, N, R = 1024, 768, 1280, 64
ctx = TpContext(dist.group.WORLD, dev, max_tokens=T_MAX, max_features=2048)
def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=dev) * scale).to(torch.bfloat16)

# microbatches of different sizes reuse the same flag and counter words: the tile indexing
# changes with the token count, only the epochs keep calls apart
for it, T in enumerate([1024, 512, 1024]):
    ms = T // world
    # ---------------- all-gather -> GEMM (+ LoRA slab), NT and NN weight layouts ----------------
    x_shard = rnd(ms, K, seed=10 * it + rank)
    s_shard = rnd(ms, R, scale=0.1, seed=100 + 10 * it + rank)
    w = rnd(N, K, scale=0.05, seed=7 + it)            # same on all ranks (a column shard in real use)
    b2 = rnd(1, N, R, scale=0.05, seed=8 + it)
    ctx.own_gather_rows(T, K).copy_(x_shard)
    ctx.own_gather2_rows(T, R).copy_(s_shard)
    y = ag_gemm(ctx, T, K, w, slab_cols=R, b2=b2, b2_adapter_rows=N)
    xs = [torch.empty_like(x_shard) for _ in range(world)]
    ss = [torch.empty_like(s_shard) for _ in range(world)]
    dist.all_gather(xs, x_shard); dist.all_gather(ss, s_shard)
    x_full, s_full = torch.cat(xs).float(), torch.cat(ss).float()
    ref = x_full @ w.float().t() + s_full @ b2[0].float().t()
    torch.cuda.synchronize(); _native.check_device_errors()
    assert_close_two_rounds(y, ref, msg=f"ag_gemm NT it{it}")
    # gathered buffer now holds every rank's rows
    assert torch.equal(ctx.gather_view(T, K).float(), x_full)

    wt = rnd(K, N, scale=0.05, seed=9 + it)
    ctx.own_gather_rows(T, K).copy_(x_shard)
    y2 = ag_gemm(ctx, T, K, wt, w_mn=True)
    torch.cuda.synchronize(); _native.check_device_errors()
    assert_close_two_rounds(y2, x_full @ wt.float(), msg=f"ag_gemm NN it{it}")

    # ---------------- GEMM -> reduce-scatter (+ LoRA slab, + residual) ----------------
    xa = rnd(T, K, seed=200 + 10 * it + rank)         # this rank's feature shard of the input
    wa = rnd(N, K, scale=0.05, seed=300 + 10 * it + rank)
    sa = rnd(T, R, scale=0.1, seed=400 + 10 * it + rank)
    res = rnd(ms, N, seed=500 + rank)
    out = gemm_rs(ctx, xa, wa, s=sa, b2=b2, b2_adapter_rows=N, residual=res)
    part = xa.float() @ wa.float().t() + sa.float() @ b2[0].float().t()
    # the kernel rounds each rank's partial to bf16 before summing
    part16 = part.to(torch.bfloat16).float()
    tot = part16.clone(); dist.all_reduce(tot)
    ref = tot[rank * ms:(rank + 1) * ms] + res.float()
    torch.cuda.synchronize(); _native.check_device_errors()
    assert_close_two_rounds(out, ref, atol=2e-2, msg=f"gemm_rs it{it}")
    if it == 0:   # the weight shard as NF4, expanded inside the fused kernels
        from lorafusion_b200.ops.nf4 import dequantize_nf4_reference, quantize_nf4
        qw, qa = quantize_nf4(w), quantize_nf4(wa)
        ctx.own_gather_rows(T, K).copy_(x_shard)
        ctx.own_gather2_rows(T, R).copy_(s_shard)
        yq = ag_gemm(ctx, T, K, qw, slab_cols=R, b2=b2, b2_adapter_rows=N)
        outq = gemm_rs(ctx, xa, qa, s=sa, b2=b2, b2_adapter_rows=N, residual=res)
        torch.cuda.synchronize(); _native.check_device_errors()
        assert_close_two_rounds(yq, x_full @ dequantize_nf4_reference(qw).float().t() + s_full @ b2[0].float().t(),
                                msg="ag_gemm NF4")
        part = xa.float() @ dequantize_nf4_reference(qa).float().t() + sa.float() @ b2[0].float().t()
        tot = part.to(torch.bfloat16).float(); dist.all_reduce(tot)
        assert_close_two_rounds(outq, tot[rank * ms:(rank + 1) * ms] + res.float(), atol=2e-2, msg="gemm_rs NF4")
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ag_gemm_and_gemm_rs_two_ranks(tmp_path):
    script = tmp_path / "child_tp.py"
    script.write_text(_CHILD)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                   PYTHONPATH=os.pathsep.join([os.getcwd(), os.environ.get("PYTHONPATH", "")]))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o[-3000:]}"


def test_world_one_degenerates_to_plain_gemm():
    """With a single rank the fused variants are ordinary GEMMs (no waits, no peers)."""
    from lorafusion_b200.parallel.tp_ops import TpContext, ag_gemm, gemm_rs
    from lorafusion_b200.utils.testing import assert_close_two_rounds

    torch.backends.cuda.matmul.allow_tf32 = False
    T, K, N = 512, 256, 512
    ctx = TpContext(None, "cuda", max_tokens=T, max_features=1024)
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    ctx.own_gather_rows(T, K).copy_(x)
    assert_close_two_rounds(ag_gemm(ctx, T, K, w), x.float() @ w.float().t(), msg="ag_gemm world 1")
    assert_close_two_rounds(gemm_rs(ctx, x, w), x.float() @ w.float().t(), msg="gemm_rs world 1")


_CHILD_MODEL = r"""
import os, torch, torch.distributed as dist
os.environ["NCCL_NVLS_ENABLE"] = "0"
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from lorafusion_b200.models.config import AdapterSpec, get_model_config
from lorafusion_b200.models.decoder import DecoderStage
from lorafusion_b200.models.tp_decoder import TpDecoderStage, _shard_rows
from lorafusion_b200.train.data import MicroBatchSpec, build_packed_batch
from lorafusion_b200.ops import _native
from lorafusion_b200.utils.testing import assert_close_two_rounds

cfg = get_model_config("tiny")
adapters = [AdapterSpec("lora_0", r=16, lora_alpha=32, dropout=0.1), AdapterSpec("lora_1", r=8, lora_alpha=16)]
for quantize, recompute in ((False, False), (False, True), (False, "auto")):   # "auto" -> the "cheap" level
    full = DecoderStage(cfg, adapters, dev, quantize=quantize, init_b_std=0.02, seed=3, recompute=False)
    spec = MicroBatchSpec([(0, [100, 37, 200]), (1, [129, 64, 100])])   # 384 + 384 = 768 tokens
    batch = build_packed_batch(spec, adapters, cfg.vocab_size, dev, seed=5)
    assert batch.num_tokens % (128 * world) == 0, batch.num_tokens
    tp = TpDecoderStage.from_full(full, dist.group.WORLD, max_tokens=batch.num_tokens, recompute=recompute)
    if recompute == "auto":
        assert tp.plan_activations(batch.num_tokens)["keep_all_gemm_outputs"] == len(tp.layers)
        assert set(tp._plan_modes(batch.num_tokens)) == {"cheap"}
    for step in range(2):          # two microbatches back to back exercise buffer reuse
        loss_full = full.forward_backward(batch)
        out, saved = tp.forward(batch)
        loss_tp, dh = tp.loss_and_grad(out, batch)
        tp.backward(saved, dh, batch)
    tp.reduce_replicated_grads()
    torch.cuda.synchronize(); _native.check_device_errors()
    assert abs(float(loss_tp) - float(loss_full)) / float(loss_full) < 1e-2, (float(loss_tp), float(loss_full))
    n = len(adapters)
    for (l, proj), fv in full.arena.views.items():
        lv = tp.arena.views[(l, proj)]
        fa, fb, la, lb = fv.stack.da, fv.stack.db, lv.stack.da, lv.stack.db
        if proj in ("qkv", "gate_up"):
            exp_a = fa
            parts = [s for _, s in fv.subs]
            exp_b = torch.stack([_shard_rows(fb[i], parts, rank, world) for i in range(n)])
        else:
            step_k = fv.K // world
            exp_a = fa[:, :, rank * step_k:(rank + 1) * step_k]
            exp_b = fb
        kw = dict(atol=3e-2, rtol=5e-2, scale_atol_by_rms=True, max_mismatch_ratio=1e-2)
        assert_close_two_rounds(la, exp_a, msg=f"dA {l} {proj} (quantize={quantize}, recompute={recompute})", **kw)
        assert_close_two_rounds(lb, exp_b, msg=f"dB {l} {proj} (quantize={quantize}, recompute={recompute})", **kw)
    if recompute is False:
        # checkpoint round trip under tensor parallelism: shards are gathered into full PEFT
        # tensors on save and cut again on load
        from lorafusion_b200.train import checkpoint as ck
        lay = ck.CheckpointLayout(tp_group=dist.group.WORLD, tp_rank=rank, tp_size=world)
        gm = torch.Generator(device=dev).manual_seed(21)   # same values on every rank
        tp.arena.m.copy_(torch.randn(tp.arena.m.shape, generator=gm, device=dev))
        out_dir = os.environ["CKPT_DIR"]
        ck.save_checkpoint(tp.arena, out_dir, lay, base_model_name="tiny")
        single = DecoderStage(cfg, adapters, dev, init_b_std=0.0, seed=11, recompute=False)
        ck.load_checkpoint(single.arena, out_dir)
        for a in range(n):   # the shards were put together in rank order: equal to the unpartitioned weights
            got, want = single.arena.export_adapter(a, "master"), full.arena.export_adapter(a, "master")
            assert got.keys() == want.keys() and all(torch.equal(got[k], want[k]) for k in want)
        before = {a: tp.arena.export_adapter(a, "m") for a in range(n)}
        work_before = tp.arena.work.clone()
        tp.arena.work.zero_(); tp.arena.m.zero_(); tp.arena.master.zero_()
        ck.load_checkpoint(tp.arena, out_dir, lay)
        for a in range(n):
            after = tp.arena.export_adapter(a, "m")
            assert all(torch.equal(after[k], before[a][k]) for k in after)
        assert torch.equal(tp.arena.work, work_before)
        del single
    del full, tp
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_stage_matches_unpartitioned_stage(tmp_path):
    script = tmp_path / "child_tp_model.py"
    script.write_text(_CHILD_MODEL)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", CKPT_DIR=str(tmp_path / "ckpt"),
                   PYTHONPATH=os.pathsep.join([os.getcwd(), os.environ.get("PYTHONPATH", "")]))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o[-4000:]}"


@pytest.mark.parametrize("world,pair", [(2, True), (2, False), (4, True)])
def test_loopback_runs_the_copy_and_reduce_warps_on_one_gpu(world, pair):
    """One GPU plays rank 0 of ``world``: peer pointers lead back to its own memory, the host
    plays the other ranks before each launch (data in place, flags raised).  The shard-push
    warps, the flag waits of the TMA producer, the partial-tile flags of the epilogue and the
    pulling reduce warps all run; results are checked against fp32 math."""
    from lorafusion_b200.ops import _native
    from lorafusion_b200.parallel.tp_ops import TpContext, ag_gemm, gemm_rs, set_pair_tp_kernels
    from lorafusion_b200.utils.testing import assert_close_two_rounds

    torch.backends.cuda.matmul.allow_tf32 = False
    dev = "cuda"
    T_MAX, K, N, R = 1024, 768, 1280, 64
    ctx = TpContext.loopback(dev, world=world, max_tokens=T_MAX, max_features=2048)
    # pair = the CTA-pair kernels where the shape allows (an even number of 128-row tiles per
    # shard: 1024 and 512 tokens at world 2, 1024 at world 4), else the single-CTA template
    set_pair_tp_kernels(pair)

    def rnd(*shape, scale=1.0, seed=0):
        g = torch.Generator(device=dev).manual_seed(seed)
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(torch.bfloat16)

    for it, T in enumerate([1024, 512, 1024]):   # sizes change: the same flag words are reused under new epochs
        ms = T // world
        # ---- all-gather -> GEMM (+ LoRA slab): the whole [T, K] operand sits in the gather buffer,
        # rows [0, ms) are "ours" (pushed by the copy warps), the rest arrived "from the peers"
        x_full, s_full = rnd(T, K, seed=10 + it), rnd(T, R, scale=0.1, seed=20 + it)
        w, b2 = rnd(N, K, scale=0.05, seed=30 + it), rnd(1, N, R, scale=0.05, seed=40 + it)
        ctx.gather_view(T, K).copy_(x_full)
        ctx.gather2_view(T, R).copy_(s_full)
        ctx.loopback_arm_gather(T)
        y = ag_gemm(ctx, T, K, w, slab_cols=R, b2=b2, b2_adapter_rows=N)
        torch.cuda.synchronize()
        _native.check_device_errors()
        assert_close_two_rounds(y, x_full.float() @ w.float().t() + s_full.float() @ b2[0].float().t(),
                                msg=f"loop-back ag_gemm it{it}")
        tps = ms // 128
        assert bool((ctx.ag_flags.tensor[:tps] == ctx.epoch).all())      # our tiles were flagged "at the peers"
        assert torch.equal(ctx.gather_view(T, K), x_full)                 # the self-push left the data intact

        # ---- GEMM -> reduce-scatter (+ slab, + residual): our partial plus the peers' stand-ins
        xa, wa = rnd(T, K, seed=50 + it), rnd(N, K, scale=0.05, seed=60 + it)
        sa, res = rnd(T, R, scale=0.1, seed=70 + it), rnd(ms, N, seed=80 + it)
        others = [rnd(T, N, seed=90 + 10 * it + r) for r in range(1, world)]
        ctx.loopback_arm_reduce(T, N, others)
        out = gemm_rs(ctx, xa, wa, s=sa, b2=b2, b2_adapter_rows=N, residual=res)
        torch.cuda.synchronize()
        _native.check_device_errors()
        mine = (xa.float() @ wa.float().t() + sa.float() @ b2[0].float().t()).to(torch.bfloat16).float()
        ref = mine[:ms] + sum(o.float()[:ms] for o in others) + res.float()
        assert_close_two_rounds(out, ref, atol=2e-2, msg=f"loop-back gemm_rs it{it}")

        if it < 2:
            # ---- the backward forms with dropout: the weight is consumed MN-major and the LoRA slab is
            # multiplied by the regenerated mask (CTA-pair kernels: in place in TMEM before the main
            # product lands on top; single-CTA template: second accumulator mixed in the epilogue)
            from lorafusion_b200.ops import lora_kernels as lk
            from lorafusion_b200.ops.philox import keep_mask

            p_drop = 0.25
            drop = lk.DropoutSpec(seed=4321 + it, stream_id=11, p=p_drop).kwargs()
            keep = keep_mask(T, N, p_drop, 4321 + it, 11).to(dev)
            dy_full, ds_full = rnd(T, K, seed=100 + it), rnd(T, R, scale=0.1, seed=110 + it)
            wt, a2 = rnd(K, N, scale=0.05, seed=120 + it), rnd(1, R, N, scale=0.05, seed=130 + it)
            ctx.gather_view(T, K).copy_(dy_full)
            ctx.gather2_view(T, R).copy_(ds_full)
            ctx.loopback_arm_gather(T)
            dx = ag_gemm(ctx, T, K, wt, w_mn=True, slab_cols=R, b2=a2, b2_adapter_rows=R, dropout_kwargs=drop)
            torch.cuda.synchronize()
            _native.check_device_errors()
            slab = torch.where(keep, ds_full.float() @ a2[0].float() / (1 - p_drop), torch.zeros((), device=dev))
            assert_close_two_rounds(dx, dy_full.float() @ wt.float() + slab, msg=f"loop-back ag_gemm dropout it{it}")
            ctx.loopback_arm_reduce(T, N, others)
            outd = gemm_rs(ctx, dy_full, wt, w_mn=True, s=ds_full, b2=a2, b2_adapter_rows=R, dropout_kwargs=drop,
                           residual=res)
            torch.cuda.synchronize()
            _native.check_device_errors()
            mine = (dy_full.float() @ wt.float() + slab).to(torch.bfloat16).float()
            assert_close_two_rounds(outd, mine[:ms] + sum(o.float()[:ms] for o in others) + res.float(), atol=2e-2,
                                    msg=f"loop-back gemm_rs dropout it{it}")

        if it == 0:
            # ---- the same two fused kernels reading their weight shard as NF4, expanded in the main loop
            from lorafusion_b200.ops.nf4 import dequantize_nf4_reference, quantize_nf4

            qw, qwt = quantize_nf4(w), quantize_nf4(rnd(K, N, scale=0.05, seed=33))
            wd, wtd = dequantize_nf4_reference(qw).float(), dequantize_nf4_reference(qwt).float()
            ctx.gather_view(T, K).copy_(x_full)
            ctx.gather2_view(T, R).copy_(s_full)
            ctx.loopback_arm_gather(T)
            yq = ag_gemm(ctx, T, K, qw, slab_cols=R, b2=b2, b2_adapter_rows=N)
            ctx.loopback_arm_gather(T)
            yq2 = ag_gemm(ctx, T, K, qwt, w_mn=True)
            ctx.loopback_arm_reduce(T, N, others)
            outq = gemm_rs(ctx, xa, qw, s=sa, b2=b2, b2_adapter_rows=N, residual=res)
            torch.cuda.synchronize()
            _native.check_device_errors()
            assert_close_two_rounds(yq, x_full.float() @ wd.t() + s_full.float() @ b2[0].float().t(),
                                    msg="loop-back ag_gemm NF4 (K-major weight)")
            assert_close_two_rounds(yq2, x_full.float() @ wtd, msg="loop-back ag_gemm NF4 (MN-major weight)")
            mine = (xa.float() @ wd.t() + sa.float() @ b2[0].float().t()).to(torch.bfloat16).float()
            assert_close_two_rounds(outq, mine[:ms] + sum(o.float()[:ms] for o in others) + res.float(), atol=2e-2,
                                    msg="loop-back gemm_rs NF4")
    set_pair_tp_kernels(True)
