"""LoRA arena layout, chunk tables, PEFT-format checkpoints and training-state resume (CPU)."""

import json

import torch
from safetensors.torch import load_file

from lorafusion_b200.models.adapters import LoRAArena
from lorafusion_b200.models.config import AdapterSpec, get_model_config
from lorafusion_b200.models import peft_io


def _arena(seed=0, **kw):
    cfg = get_model_config("tiny")
    adapters = [AdapterSpec("lora_0", r=16), AdapterSpec("lora_1", r=8, lora_alpha=16, dropout=0.05,
                                                         target_modules=("q_proj", "v_proj", "down_proj"))]
    return LoRAArena(cfg, adapters, range(cfg.num_layers), "cpu", init_b_std=0.02, seed=seed, **kw), cfg


def test_layout_block_diagonal_and_padding_stay_zero():
    arena, cfg = _arena()
    v = arena.views[(0, "qkv")]
    assert (v.K, v.N, v.R) == (512, cfg.qkv_size, 64) and v.slot == 16
    st = v.stack
    # adapter 0 (r=16, all targets): A rows 0:48 used; B block diagonal
    assert float(st.a[0, 48:].abs().max()) == 0 and float(st.a[0, :48].abs().min()) > 0
    q, kv = cfg.q_size, cfg.kv_size
    assert float(st.b[0, :q, 16:].abs().max()) == 0            # q rows only use cols 0:16
    assert float(st.b[0, q:q + kv, :16].abs().max()) == 0      # k rows only use cols 16:32
    assert float(st.b[0, q + kv:, 32:48].abs().min()) > 0      # v rows use cols 32:48
    # adapter 1 (r=8, q and v only): k slot untouched
    assert float(st.a[1, 16:32].abs().max()) == 0 and float(st.a[1, 8:16].abs().max()) == 0
    assert float(st.b[1, q:q + kv].abs().max()) == 0


def test_chunk_table_covers_each_adapter_exactly():
    arena, _ = _arena()
    for adapter in range(2):
        chunks = arena.chunk_table(adapter).tolist()
        covered = torch.zeros(arena.numel, dtype=torch.int32)
        trainable = torch.zeros(arena.numel, dtype=torch.bool)
        state_seen = torch.zeros(arena.state_numel, dtype=torch.int32)
        for off, rows, ld, c0, cols, state in chunks:
            covered[off:off + rows * ld] += 1
            blk = torch.zeros(rows, ld, dtype=torch.bool)
            blk[:, c0:c0 + cols] = True
            trainable[off:off + rows * ld] |= blk.view(-1)
            if cols:
                assert state % 4 == 0
                state_seen[state:state + rows * cols] += 1
                # the dense fp32 master mirrors the trainable window of the bf16 working copy
                win = arena.work[off:off + rows * ld].view(rows, ld)[:, c0:c0 + cols].float()
                assert torch.equal(arena.master[state:state + rows * cols].view(rows, cols), win)
        lo, hi = arena.state_range[adapter]
        assert int(state_seen.max()) == 1 and int(state_seen[:lo].sum()) == 0 and int(state_seen[hi:].sum()) == 0
        assert int(state_seen.sum()) == arena.trainable_numel(adapter)
        n = arena.num_adapters
        expect = torch.zeros(arena.numel, dtype=torch.bool)
        for v in arena.views.values():
            a0 = v.a_offset + adapter * v.R * v.K
            b0 = v.b_offset + adapter * v.N * v.R
            expect[a0:a0 + v.R * v.K] = True
            expect[b0:b0 + v.N * v.R] = True
        assert torch.equal(covered > 0, expect) and int(covered.max()) == 1
        assert int(trainable.sum()) == arena.trainable_numel(adapter)
        # every initialised (non-zero) weight lies inside the trainable window
        nz = arena.work != 0
        assert not bool((nz & expect & ~trainable).any())
    assert arena.trainable_numel(0) == sum(16 * (len(v.subs) * v.K + v.N) for v in arena.views.values())


def test_peft_checkpoint_roundtrip(tmp_path):
    arena, cfg = _arena(seed=1)
    out = peft_io.save_adapter(arena, 1, tmp_path / "lora_1", base_model_name="tiny")
    conf = json.loads((out / "adapter_config.json").read_text())
    assert conf["peft_type"] == "LORA" and conf["r"] == 8 and conf["lora_alpha"] == 16
    assert conf["target_modules"] == ["down_proj", "q_proj", "v_proj"]
    raw = load_file(str(out / "adapter_model.safetensors"))
    key = "base_model.model.model.layers.1.self_attn.v_proj.lora_B.weight"
    assert raw[key].shape == (cfg.kv_size, 8)
    assert raw["base_model.model.model.layers.0.mlp.down_proj.lora_A.weight"].shape == (8, cfg.intermediate_size)
    assert not any("k_proj" in k for k in raw)
    other, _ = _arena(seed=2)
    before = other.work.clone()
    peft_io.load_adapter(other, 1, out)
    for k, t in arena.export_adapter(1).items():
        assert torch.allclose(other.export_adapter(1)[k], t.to(torch.bfloat16).float())
    v = other.views[(0, "o")]
    n_a = other.num_adapters * v.R * v.K
    # adapter 0 untouched
    assert torch.equal(other.work[v.a_offset:v.a_offset + v.R * v.K], before[v.a_offset:v.a_offset + v.R * v.K])
    assert peft_io.load_adapter_config(out).scaling == 2.0 and n_a > 0


def test_training_state_roundtrip(tmp_path):
    arena, _ = _arena(seed=3)
    arena.m.normal_()
    arena.v.uniform_()
    arena.steps[0] = 7
    peft_io.save_training_state(arena, 0, tmp_path / "state0.pt", data_cursor=123, extra={"lr": 1e-4})
    other, _ = _arena(seed=4)
    meta = peft_io.load_training_state(other, 0, tmp_path / "state0.pt")
    assert meta == {"step": 7, "data_cursor": 123, "extra": {"lr": 1e-4}} and other.steps[0] == 7
    sl = slice(*arena.state_range[0])
    assert torch.equal(other.m[sl], arena.m[sl]) and torch.equal(other.master[sl], arena.master[sl])
    for k, t in arena.export_adapter(0).items():
        assert torch.equal(other.export_adapter(0)[k], t)
    st, ot = arena.stack(0, "qkv"), other.stack(0, "qkv")
    assert torch.equal(st.a[0], ot.a[0]) and torch.equal(st.b[0], ot.b[0])
    # adapter 1's state was not touched
    sl1 = slice(*arena.state_range[1])
    assert not torch.equal(other.m[sl1], arena.m[sl1])


def test_adam_work_items_cover_every_element_exactly_once():
    from lorafusion_b200.ops.elementwise import build_adam_work_items

    arena, _ = _arena()
    for adapter in range(2):
        rows = arena._chunk_rows[adapter]
        for world in (1, 3):
            seen = [torch.zeros(r[1] * r[2], dtype=torch.int32) for r in rows]
            for rank in range(world):
                items = build_adam_work_items(rows, rank=rank, world=world, unit=1024)
                assert items.dtype == torch.int32 and items.shape[1] == 3
                for ci, first, count in items.tolist():
                    assert 0 < count <= 1024 and first % 4 == 0 and count % 4 == 0
                    seen[ci][first:first + count] += 1
            assert all(int(s.min()) == 1 and int(s.max()) == 1 for s in seen if s.numel())
    # regions with odd offsets keep working on the scalar path with smaller pieces
    odd = build_adam_work_items([(4301, 10, 30, 3, 10, 2600)], unit=1024).tolist()
    assert sum(c for _, _, c in odd) == 300 and all(c <= 256 for _, _, c in odd)
