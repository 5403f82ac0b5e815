"""Fused gradient reduce + AdamW + weight broadcast kernel.

On one GPU the data-parallel ranks are emulated by running the kernel once per rank, one
after another, over all ranks' arenas with the cross-rank flags switched off (kernels that
wait on one another must never be launched separately on one GPU).  The 2-GPU test launches
real ranks as child processes with NCCL's NVLS off and plain peer loads in the kernel.
"""

import os
import socket
import subprocess
import sys

import pytest
import torch

from lorafusion_b200.models.adapters import LoRAArena
from lorafusion_b200.models.config import AdapterSpec, get_model_config
from lorafusion_b200.utils.testing import assert_close

pytestmark = pytest.mark.gpu


def _arena(seed=0):
    cfg = get_model_config("tiny")
    adapters = [AdapterSpec("a", r=16), AdapterSpec("b", r=8, target_modules=("q_proj", "v_proj", "down_proj"))]
    return LoRAArena(cfg, adapters, range(cfg.num_layers), "cuda", init_b_std=0.02, seed=seed)


@pytest.mark.parametrize("world", [1, 4])
def test_emulated_ranks_match_allreduce_plus_adamw(world):
    from lorafusion_b200.parallel.dp_sync import launch_allreduce_adam

    arenas = [_arena() for _ in range(world)]
    ref = _arena()
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.05)
    for step in range(1, 3):
        g = torch.Generator(device="cuda").manual_seed(step)
        total = torch.zeros_like(ref.grad)
        for a in arenas:
            a.grad.copy_(torch.randn(a.numel, generator=g, device="cuda"))
            total += a.grad
        for adapter in range(2):
            ref.grad.copy_(total)
            ref.adam_step(adapter, grad_scale=0.25, **hp)
            for r, a in enumerate(arenas):
                launch_allreduce_adam(
                    chunks=a.chunk_table(adapter), grad_ptrs=[x.grad.data_ptr() for x in arenas],
                    work_ptrs=[x.work.data_ptr() for x in arenas], grad_mc=0, work_mc=0, master=a.master, m=a.m,
                    v=a.v, flag_ptrs=None, done_counter=None, rank=r, world=world, epoch=0, sync=False,
                    use_multimem=False, step=step, grad_scale=0.25, device="cuda", **hp)
            # restore the other adapter's gradients consumed from `total` bookkeeping
            chunks = ref.chunk_table(adapter).cpu()
            for off, rows, ld, _, _, _ in chunks.tolist():
                total[off:off + rows * ld] = 0
                for a in arenas:
                    assert float(a.grad[off:off + rows * ld].abs().max()) == 0.0
    for a in arenas:
        assert_close(a.work, ref.work, msg="bf16 working copies after the fused step")
    # every optimizer-state element is owned by exactly one rank: stitched masters == reference
    stitched = torch.zeros_like(ref.master)
    touched = torch.zeros_like(ref.master, dtype=torch.bool)
    base = _arena()
    for a in arenas:
        diff = a.master != base.master
        stitched[diff] = a.master[diff]
        touched |= diff
    assert_close(stitched[touched], ref.master[touched], rtol=1e-5, atol=1e-6, msg="sharded master weights")


@pytest.mark.parametrize("world", [2, 4])
def test_checkpoint_after_fused_steps_equals_allreduce_plus_adamw(world, tmp_path):
    """Three fused steps on emulated ranks; the optimizer state is stitched from its owners the
    way ``gather_owned_state`` does with an all-reduce (masked sum), saved from rank 0 and loaded
    into a fresh single-rank arena: weights, master and both moments equal the reference that ran
    sum-of-gradients + the plain Adam kernel."""
    from lorafusion_b200.parallel.dp_sync import launch_allreduce_adam
    from lorafusion_b200.train import checkpoint as ck

    arenas = [_arena() for _ in range(world)]
    ref = _arena()
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.05)
    for step in range(1, 4):
        g = torch.Generator(device="cuda").manual_seed(10 + step)
        total = torch.zeros_like(ref.grad)
        for a in arenas:
            a.grad.copy_(torch.randn(a.numel, generator=g, device="cuda"))
            total += a.grad
        for adapter in range(2):
            ref.grad.copy_(total)
            ref.adam_step(adapter, grad_scale=1.0 / world, **hp)
            for off, rows, ld, _, _, _ in ref.chunk_table(adapter).cpu().tolist():
                total[off:off + rows * ld] = 0
            for r, a in enumerate(arenas):
                launch_allreduce_adam(
                    chunks=a.chunk_table(adapter), grad_ptrs=[x.grad.data_ptr() for x in arenas],
                    work_ptrs=[x.work.data_ptr() for x in arenas], grad_mc=0, work_mc=0, master=a.master, m=a.m,
                    v=a.v, flag_ptrs=None, done_counter=None, rank=r, world=world, epoch=0, sync=False,
                    use_multimem=False, step=step, grad_scale=1.0 / world, device="cuda", **hp)
                a.steps[adapter] = step
    # rank 0 alone holds stale state for the slices it does not own
    lo, hi = arenas[0].state_range[0]
    assert not torch.equal(arenas[0].m[lo:hi], ref.m[lo:hi])
    for adapter in range(2):
        lo, hi = ref.state_range[adapter]
        for name in ("master", "m", "v"):
            acc = torch.zeros(hi - lo, device="cuda")
            for r, a in enumerate(arenas):
                acc += getattr(a, name)[lo:hi].masked_fill(~a.owned_state_mask(adapter, r, world), 0.0)
            getattr(arenas[0], name)[lo:hi].copy_(acc)
    ck.save_checkpoint(arenas[0], tmp_path, base_model_name="tiny")
    fresh = _arena(seed=5)
    metas = ck.load_checkpoint(fresh, tmp_path)
    assert [m["step"] for m in metas] == [3, 3]
    for adapter in range(2):
        for name in ("master", "m", "v"):
            got, want = fresh.export_adapter(adapter, name), ref.export_adapter(adapter, name)
            for k in want:
                assert_close(got[k], want[k], rtol=1e-6, atol=1e-7, msg=f"{name} {k}")
        got, want = fresh.export_adapter(adapter, "work"), ref.export_adapter(adapter, "work")
        for k in want:
            assert_close(got[k], want[k], msg=f"work {k}")


def test_layer_group_launches_on_a_side_stream_equal_one_whole_launch():
    """The sync of a step may be launched group of layers by group of layers (so that it can
    overlap the rest of the backward): same weights, state and cleared gradients as one launch."""
    from lorafusion_b200.parallel.dp_sync import FusedGradSync
    from lorafusion_b200.parallel.symmetric import SymmetricAllocator
    from lorafusion_b200.train.trainer import OptimizerConfig

    cfg = get_model_config("tiny")
    adapters = [AdapterSpec("a", r=16), AdapterSpec("b", r=8, target_modules=("q_proj", "v_proj", "down_proj"))]
    opt = OptimizerConfig(lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.05)
    arenas, syncs = [], []
    for _ in range(2):
        alloc = SymmetricAllocator("cuda", None)
        ar = LoRAArena(cfg, adapters, range(cfg.num_layers), "cuda", init_b_std=0.02, seed=0, shared_alloc=alloc)
        arenas.append(ar)
        syncs.append(FusedGradSync(ar, alloc, None, opt))
    side = torch.cuda.Stream()
    syncs[0].trace = torch.zeros(3 * 4096, dtype=torch.int64, device="cuda")   # in-kernel time stamps
    for step in range(1, 3):
        g = torch.Generator(device="cuda").manual_seed(step)
        grad = torch.randn(arenas[0].numel, generator=g, device="cuda")
        for ar in arenas:
            ar.grad.copy_(grad)
        for a in range(2):
            syncs[0].reduce_and_step(a, grad_scale=0.5)
            n = syncs[1].begin_step(a)
            for layers in ((1, 2), (0, 1)):       # the order a backward pass completes them in
                ev = torch.cuda.Event()
                ev.record()
                side.wait_event(ev)
                with torch.cuda.stream(side):
                    syncs[1].reduce_and_step(a, grad_scale=0.5, layers=layers, step=n)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        assert arenas[1].steps == arenas[0].steps == [step, step]
        for name in ("work", "master", "m", "v", "grad"):
            assert torch.equal(getattr(arenas[0], name), getattr(arenas[1], name)), (step, name)
    assert float(arenas[1].grad.abs().max()) == 0.0
    from lorafusion_b200.parallel.dp_sync import summarize_sync_trace

    tr = summarize_sync_trace(syncs[0].trace, syncs[0].last_num_items)
    assert tr["end_ns"] > tr["start_ns"] > 0 and 0.0 < tr["span_us"] < 1e5
    assert 0.0 <= tr["max_wait_for_peers_us"] <= tr["span_us"] and tr["mean_work_us"] > 0.0


_CHILD = r"""
import os, sys, torch, torch.distributed as dist
os.environ["NCCL_NVLS_ENABLE"] = "0"
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from lorafusion_b200.models.adapters import LoRAArena
from lorafusion_b200.models.config import AdapterSpec, get_model_config
from lorafusion_b200.parallel.dp_sync import FusedGradSync
from lorafusion_b200.parallel.symmetric import SymmetricAllocator
from lorafusion_b200.train.trainer import OptimizerConfig
from lorafusion_b200.ops import _native
cfg = get_model_config("tiny")
adapters = [AdapterSpec("a", r=16), AdapterSpec("b", r=8)]
alloc = SymmetricAllocator(f"cuda:{rank}", dist.group.WORLD)
arena = LoRAArena(cfg, adapters, range(cfg.num_layers), f"cuda:{rank}", init_b_std=0.02, seed=0, shared_alloc=alloc)
ref = LoRAArena(cfg, adapters, range(cfg.num_layers), f"cuda:{rank}", init_b_std=0.02, seed=0)
opt = OptimizerConfig(lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.05)
sync = FusedGradSync(arena, alloc, dist.group.WORLD, opt, use_multimem=False)
for step in range(1, 4):
    g = torch.Generator(device="cuda").manual_seed(100 * step + rank)
    arena.grad.copy_(torch.randn(arena.numel, generator=g, device="cuda"))
    total = arena.grad.clone()
    dist.all_reduce(total)
    for adapter in range(2):
        ref.grad.copy_(total)
        ref.adam_step(adapter, lr=opt.lr, beta1=opt.beta1, beta2=opt.beta2, eps=opt.eps,
                      weight_decay=opt.weight_decay, grad_scale=0.5)
        sync.reduce_and_step(adapter, grad_scale=0.5)
    torch.cuda.synchronize()
    _native.check_device_errors()
    err = (arena.work.float() - ref.work.float()).abs().max().item()
    assert err < 1e-2, f"rank {rank} step {step}: work copy differs by {err}"
    assert arena.grad.abs().max().item() == 0.0
# one more step, launched layer group by layer group on a side stream
side = torch.cuda.Stream()
g = torch.Generator(device="cuda").manual_seed(900 + rank)
arena.grad.copy_(torch.randn(arena.numel, generator=g, device="cuda"))
total = arena.grad.clone()
dist.all_reduce(total)
for adapter in range(2):
    ref.grad.copy_(total)
    ref.adam_step(adapter, lr=opt.lr, beta1=opt.beta1, beta2=opt.beta2, eps=opt.eps,
                  weight_decay=opt.weight_decay, grad_scale=0.5)
    n = sync.begin_step(adapter)
    for layers in ((1, 2), (0, 1)):
        ev = torch.cuda.Event(); ev.record(); side.wait_event(ev)
        with torch.cuda.stream(side):
            sync.reduce_and_step(adapter, grad_scale=0.5, layers=layers, step=n)
torch.cuda.current_stream().wait_stream(side)
torch.cuda.synchronize()
_native.check_device_errors()
err = (arena.work.float() - ref.work.float()).abs().max().item()
assert err < 1e-2, f"rank {rank} grouped step: work copy differs by {err}"
assert arena.grad.abs().max().item() == 0.0
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_real_ranks_over_peer_memory(tmp_path):
    script = tmp_path / "child.py"
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


def test_peer_that_never_signals_ends_in_an_error_status_not_a_hang():
    """The fused sync kernel waits for every rank's "gradients ready" flag.  Here rank 1 does
    not exist: its flag is never set, the (shortened) wait runs out, the kernel records the
    failure and returns, the host reads the status, and the context stays usable."""
    from lorafusion_b200.ops import _native
    from lorafusion_b200.parallel.dp_sync import launch_allreduce_adam

    a, ghost = _arena(), _arena(seed=1)
    before = a.work.clone()
    a.grad.normal_()
    my_pad = torch.zeros(16, dtype=torch.int32, device="cuda")      # what peers would write to
    ghost_pad = torch.zeros(16, dtype=torch.int32, device="cuda")   # what this rank writes to
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0)
    _native.check_device_errors()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    launch_allreduce_adam(
        chunks=a.chunk_table(0), grad_ptrs=[a.grad.data_ptr(), ghost.grad.data_ptr()],
        work_ptrs=[a.work.data_ptr(), ghost.work.data_ptr()], grad_mc=0, work_mc=0, master=a.master, m=a.m,
        v=a.v, flag_ptrs=[my_pad.data_ptr(), ghost_pad.data_ptr()], done_counter=done, rank=0, world=2, epoch=1,
        sync=True, use_multimem=False, step=1, grad_scale=1.0, device="cuda", wait_ms=200, **hp)
    t1.record()
    with pytest.raises(RuntimeError, match="peer flag"):
        _native.check_device_errors()
    assert 150.0 < t0.elapsed_time(t1) < 5000.0           # gave up after the limit, did not spin on
    assert int(ghost_pad[0]) == 1                          # it did announce itself to the peer
    assert torch.equal(a.work, before)                     # and applied nothing
    # the status word was cleared by the read; the same context runs the single-rank path fine
    launch_allreduce_adam(
        chunks=a.chunk_table(0), grad_ptrs=[a.grad.data_ptr()], work_ptrs=[a.work.data_ptr()], grad_mc=0,
        work_mc=0, master=a.master, m=a.m, v=a.v, flag_ptrs=None, done_counter=None, rank=0, world=1, epoch=0,
        sync=False, use_multimem=False, step=1, grad_scale=1.0, device="cuda", **hp)
    _native.check_device_errors()
    assert not torch.equal(a.work, before)
