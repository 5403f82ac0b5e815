"""Checkpoints under data / tensor / pipeline parallel layouts, as far as a CPU can check them:
ownership masks of the sharded optimizer state, the masked-sum gather on gloo ranks, the
tensor-parallel shard <-> full mapping, and the pipeline-stage merge into one PEFT directory."""

import os
import socket
from dataclasses import replace

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from safetensors.torch import load_file

from lorafusion_b200.models import peft_io
from lorafusion_b200.models.adapters import LoRAArena
from lorafusion_b200.models.config import AdapterSpec, get_model_config
from lorafusion_b200.ops.elementwise import build_adam_work_items
from lorafusion_b200.train import checkpoint as ck

ADAPTERS = [AdapterSpec("lora_0", r=16), AdapterSpec("lora_1", r=8, target_modules=("q_proj", "v_proj", "down_proj"))]


def _arena(cfg=None, layers=None, seed=0):
    cfg = cfg or get_model_config("tiny")
    layers = range(cfg.num_layers) if layers is None else layers
    return LoRAArena(cfg, ADAPTERS, layers, "cpu", init_b_std=0.02, seed=seed)


def test_owned_state_masks_partition_the_state_and_match_the_kernel_split():
    arena = _arena()
    for adapter in range(2):
        lo, hi = arena.state_range[adapter]
        for world in (1, 2, 3, 4):
            masks = [arena.owned_state_mask(adapter, r, world) for r in range(world)]
            total = torch.stack([m.int() for m in masks]).sum(0)
            # every trainable element has exactly one owner; alignment gaps of the state layout have none
            used = torch.zeros(hi - lo, dtype=torch.bool)
            for _, rows, ld, col0, cols, state in arena._chunk_rows[adapter]:
                used[state - lo:state - lo + rows * cols] = cols > 0
            assert torch.equal(total, used.int())
            # the same elements the fused kernel's work items of that rank touch
            for r in range(world):
                mine = torch.zeros(hi - lo, dtype=torch.bool)
                items = build_adam_work_items(arena._chunk_rows[adapter], rank=r, world=world, unit=256).tolist()
                for ci, first, count in items:
                    _, rows, ld, col0, cols, state = arena._chunk_rows[adapter][ci]
                    e = torch.arange(first, first + count)
                    row, col = e // ld, e % ld
                    ok = (col >= col0) & (col < col0 + cols)
                    mine[(state - lo + row * cols + col - col0)[ok]] = True
                assert torch.equal(mine, masks[r])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gather_worker(rank, world, port, tmp, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        arena = _arena()
        g = torch.Generator().manual_seed(5)
        upd = {n: torch.randn(arena.state_numel, generator=g) for n in ("master", "m", "v")}
        # what the fused kernel leaves behind: only the owner of an element has its new value
        for adapter in range(2):
            lo, hi = arena.state_range[adapter]
            mask = arena.owned_state_mask(adapter, rank, world)
            for n in upd:
                getattr(arena, n)[lo:hi][mask] += upd[n][lo:hi][mask]
            arena.steps[adapter] = 3
        layout = ck.CheckpointLayout(dp_group=dist.group.WORLD, dp_rank=rank, dp_size=world, fused_dp=True)
        ck.save_checkpoint(arena, tmp, layout, base_model_name="tiny", data_cursors=[12, 6], extra={"microbatches": 9})
        q.put((rank, True))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_fused_dp_state_is_stitched_from_its_owners_before_saving(tmp_path):
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, world, port, str(tmp_path), q)) for r in range(world)]
    for p in procs:
        p.start()
    for _ in range(world):
        q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # expected: a single-rank arena with the whole update applied
    want = _arena()
    g = torch.Generator().manual_seed(5)
    upd = {n: torch.randn(want.state_numel, generator=g) for n in ("master", "m", "v")}
    for adapter in range(2):
        lo, hi = want.state_range[adapter]
        used = torch.stack([want.owned_state_mask(adapter, 0, 1)]).any(0)
        for n in upd:
            getattr(want, n)[lo:hi][used] += upd[n][lo:hi][used]
    got = _arena(seed=9)
    metas = ck.load_checkpoint(got, tmp_path)
    assert metas[0] == {"step": 3, "data_cursor": 12, "extra": {"microbatches": 9}} and metas[1]["data_cursor"] == 6
    for adapter in range(2):
        for n in ("master", "m", "v"):
            a, b = got.export_adapter(adapter, n), want.export_adapter(adapter, n)
            assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a), n
        w = got.export_adapter(adapter, "work")
        assert all(torch.equal(w[k], t.to(torch.bfloat16)) for k, t in want.export_adapter(adapter, "master").items())


def test_tensor_parallel_shards_round_trip_and_resume_under_another_degree(tmp_path):
    from lorafusion_b200.models.tp_decoder import local_config

    cfg = get_model_config("tiny")
    full = _arena(cfg)
    full.m.normal_()
    full.v.uniform_()
    ck.save_checkpoint(full, tmp_path / "full", base_model_name="tiny", data_cursors=[4, 4])
    for tp in (2, 4):
        if cfg.num_heads % tp or cfg.num_kv_heads % tp or cfg.intermediate_size % (tp * 256):
            continue
        locals_ = []
        for r in range(tp):
            arena = _arena(local_config(cfg, tp), seed=3)
            ck.load_checkpoint(arena, tmp_path / "full", ck.CheckpointLayout(tp_rank=r, tp_size=tp))
            locals_.append(arena)
        for adapter in range(2):
            for src in ("master", "m", "v"):
                back = ck.tp_unshard([a.export_adapter(adapter, src) for a in locals_])
                want = full.export_adapter(adapter, src)
                assert back.keys() == want.keys()
                assert all(torch.equal(back[k], want[k]) for k in want), (tp, src)
        # shard shapes: B of column-parallel and A of row-parallel modules are cut, the rest replicated
        e0 = locals_[0].export_adapter(0)
        assert e0["layers.0.q_proj.lora_B"].shape == (cfg.q_size // tp, 16)
        assert e0["layers.0.q_proj.lora_A"].shape == (16, cfg.hidden_size)
        assert e0["layers.0.down_proj.lora_A"].shape == (16, cfg.intermediate_size // tp)
        assert e0["layers.0.down_proj.lora_B"].shape == (cfg.hidden_size, 16)


def _pp_worker(rank, world, port, tmp, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = get_model_config("tiny")
        per = cfg.num_layers // world
        arena = _arena(cfg, range(rank * per, (rank + 1) * per), seed=1)
        arena.steps = [2, 2]
        ck.save_checkpoint(arena, tmp, ck.CheckpointLayout(pp_rank=rank, pp_size=world), base_model_name="tiny")
        q.put(rank)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_pipeline_stages_merge_into_one_peft_directory(tmp_path):
    cfg = get_model_config("tiny")
    world = 2
    assert cfg.num_layers % world == 0
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pp_worker, args=(r, world, port, str(tmp_path), q)) for r in range(world)]
    for p in procs:
        p.start()
    for _ in range(world):
        q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    raw = load_file(str(tmp_path / "lora_0" / "adapter_model.safetensors"))
    layers = {int(k.split(".layers.")[1].split(".")[0]) for k in raw}
    assert layers == set(range(cfg.num_layers)) and not (tmp_path / "lora_0" / ".parts").exists()
    # a whole-model arena and a single stage both load from the merged directory
    whole = _arena(cfg, seed=8)
    metas = ck.load_checkpoint(whole, tmp_path)
    assert metas[0]["step"] == 2
    per = cfg.num_layers // world
    for rank in range(world):
        src = _arena(cfg, range(rank * per, (rank + 1) * per), seed=1)
        for k, t in src.export_adapter(0).items():
            assert torch.equal(whole.export_adapter(0)[k], t)
    stage1 = _arena(cfg, range(per, 2 * per), seed=4)
    ck.load_checkpoint(stage1, tmp_path, ck.CheckpointLayout(pp_rank=1, pp_size=2))
    assert all(torch.equal(stage1.export_adapter(1, "master")[k], t) for k, t in
               _arena(cfg, range(per, 2 * per), seed=1).export_adapter(1, "master").items())
