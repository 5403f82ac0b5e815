"""Adapter checkpoints that are correct under every dp x pp x tp layout.

What makes a multi-rank checkpoint differ from the single-rank one of ``models/peft_io.py``:

* **Fused data-parallel gradient sync** keeps the optimizer state ZeRO-1 style: the kernel of
  ``csrc/comm/allreduce_adam.cu`` updates ``master`` / ``m`` / ``v`` only on the rank that owns a
  slice and broadcasts only the bf16 weights.  Before saving, every element is taken from its
  owner (:meth:`LoRAArena.gather_owned_state`, one masked all-reduce per tensor).
* **Tensor parallelism** shards one LoRA factor per projection with the base weight: ``B`` of
  the column-parallel q|k|v and gate|up by rows, ``A`` of the row-parallel o and down by columns;
  the other factor is replicated.  Shards are all-gathered into full tensors on save and cut
  again on load, so a checkpoint can be resumed under another tensor-parallel degree.
* **Pipeline parallelism** gives every stage its own layers.  Each stage writes a part file and
  one rank merges the parts into ONE PEFT directory per adapter that ``PeftModel`` can load.

The reference saves nothing (``SAVE_MODEL`` is parsed and ignored,
``benchmarks_paper/scripts/run_single.sh:54,219-221``); the format is PEFT's because its adapters
are PEFT adapters named ``lora_{i}`` (``lorafusion/train/training_utils.py:604-619``).

On disk::

    <dir>/<adapter name>/adapter_config.json
    <dir>/<adapter name>/adapter_model.safetensors     all layers, bf16, PEFT key names
    <dir>/<adapter name>/training_state.pt             fp32 master, m, v by layer / module + step + cursor
"""

from __future__ import annotations

import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..models import peft_io
from ..models.adapters import LoRAArena

COLUMN_PARALLEL = {"q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"}   # B sharded by rows
ROW_PARALLEL = {"o_proj", "down_proj"}                                     # A sharded by columns


@dataclass
class CheckpointLayout:
    """Where this rank sits; the defaults describe a single process."""

    dp_group: object = None
    dp_rank: int = 0
    dp_size: int = 1
    fused_dp: bool = False      # optimizer state sharded over dp by the fused sync kernel
    tp_group: object = None
    tp_rank: int = 0
    tp_size: int = 1
    pp_rank: int = 0
    pp_size: int = 1

    @property
    def is_writer(self) -> bool:
        """One rank per pipeline stage holds complete tensors to write."""
        return self.dp_rank == 0 and self.tp_rank == 0

    @classmethod
    def from_parallel_state(cls, state, *, fused_dp: bool) -> "CheckpointLayout":
        lay = state.layout
        return cls(dp_group=state.dp_group, dp_rank=state.dp_rank, dp_size=lay.dp, fused_dp=fused_dp,
                   tp_group=state.tp_group, tp_rank=state.tp_rank, tp_size=lay.tp,
                   pp_rank=state.pp_rank, pp_size=lay.pp)


# ---------------------------------------------------------------------------------------------
# tensor-parallel shards <-> full tensors
# ---------------------------------------------------------------------------------------------
def _shard_dim(key: str) -> Optional[int]:
    """Dimension along which the tensor under ``key`` is sharded over tp (None = replicated)."""
    _, _, module, which = key.split(".")
    if module in COLUMN_PARALLEL and which == "lora_B":
        return 0
    if module in ROW_PARALLEL and which == "lora_A":
        return 1
    return None


def tp_unshard(per_rank: Sequence[dict]) -> dict:
    """Full tensors from the dictionaries of all tensor-parallel ranks, in rank order."""
    out = {}
    for key, t0 in per_rank[0].items():
        dim = _shard_dim(key)
        out[key] = t0 if dim is None else torch.cat([d[key] for d in per_rank], dim=dim)
    return out


def tp_shard(full: dict, tp_rank: int, tp_size: int) -> dict:
    """This rank's part of full tensors."""
    if tp_size == 1:
        return dict(full)
    out = {}
    for key, t in full.items():
        dim = _shard_dim(key)
        if dim is None:
            out[key] = t
        else:
            if t.shape[dim] % tp_size:
                raise ValueError(f"{key}: size {t.shape[dim]} is not divisible by tp={tp_size}")
            step = t.shape[dim] // tp_size
            out[key] = t.narrow(dim, tp_rank * step, step).contiguous()
    return out


def tp_gather(tensors: dict, layout: CheckpointLayout) -> dict:
    """Collective over the tensor-parallel group: full tensors on every rank.  One all-gather of
    the flattened dictionary (every rank holds the same keys and local shapes)."""
    if layout.tp_size == 1:
        return tensors
    keys = list(tensors)
    flat = torch.cat([tensors[k].reshape(-1).float() for k in keys]) if keys else torch.zeros(0)
    gathered = torch.empty((layout.tp_size, flat.numel()), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(gathered, flat.contiguous(), group=layout.tp_group)
    per_rank = []
    for r in range(layout.tp_size):
        d, off = {}, 0
        for k in keys:
            n = tensors[k].numel()
            d[k] = gathered[r, off:off + n].view(tensors[k].shape)
            off += n
        per_rank.append(d)
    return tp_unshard(per_rank)


# ---------------------------------------------------------------------------------------------
# save / load
# ---------------------------------------------------------------------------------------------
def _barrier() -> None:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def save_checkpoint(arena: LoRAArena, out_dir: str | Path, layout: Optional[CheckpointLayout] = None, *,
                    base_model_name: str = "", data_cursors: Optional[Sequence[int]] = None,
                    extra: Optional[dict] = None, with_training_state: bool = True) -> Path:
    """Collective over all ranks of the job: write one PEFT directory per adapter under
    ``out_dir``, plus ``training_state.pt`` (unless ``with_training_state`` is False or the
    arena has no optimizer state).  ``data_cursors[i]`` = samples adapter ``i`` has consumed;
    ``extra`` is stored verbatim with every adapter's state."""
    layout = layout or CheckpointLayout()
    out_dir = Path(out_dir)
    has_state = with_training_state and arena.master is not None
    if layout.fused_dp and layout.dp_size > 1 and arena.master is not None:
        arena.gather_owned_state(layout.dp_group, layout.dp_rank, layout.dp_size)
    for i, spec in enumerate(arena.adapters):
        sources = ["master" if arena.master is not None else "work"] + (["m", "v"] if has_state else [])
        full = {src: tp_gather(arena.export_adapter(i, src), layout) for src in sources}
        if not layout.is_writer:
            continue
        weights = full[sources[0]]
        state = {"master": weights, "m": full["m"], "v": full["v"]} if has_state else None
        cursor = int(data_cursors[i]) if data_cursors is not None else 0
        if layout.pp_size == 1:
            d = peft_io.write_adapter_tensors(weights, spec, out_dir / spec.name, base_model_name=base_model_name)
            if state is not None:
                peft_io.write_training_state(state, d / "training_state.pt", step=arena.steps[i], data_cursor=cursor,
                                             extra=extra)
        else:
            parts = out_dir / spec.name / ".parts"
            parts.mkdir(parents=True, exist_ok=True)
            torch.save({"weights": {k: t.cpu() for k, t in weights.items()},
                        "state": None if state is None else {n: {k: t.cpu() for k, t in d.items()}
                                                             for n, d in state.items()},
                        "step": arena.steps[i], "data_cursor": cursor}, str(parts / f"stage{layout.pp_rank}.pt"))
    _barrier()
    if layout.pp_size > 1 and layout.is_writer and layout.pp_rank == 0:
        for spec in arena.adapters:
            parts = out_dir / spec.name / ".parts"
            weights, state, step, cursor = {}, None, 0, 0
            for s in range(layout.pp_size):
                part = torch.load(str(parts / f"stage{s}.pt"), map_location="cpu", weights_only=False)
                weights.update(part["weights"])
                if part["state"] is not None:
                    state = state or {"master": {}, "m": {}, "v": {}}
                    for n in state:
                        state[n].update(part["state"][n])
                step, cursor = max(step, int(part["step"])), max(cursor, int(part["data_cursor"]))
            d = peft_io.write_adapter_tensors(weights, spec, out_dir / spec.name, base_model_name=base_model_name)
            if state is not None:
                peft_io.write_training_state(state, d / "training_state.pt", step=step, data_cursor=cursor, extra=extra)
            shutil.rmtree(parts)
    _barrier()
    return out_dir


def load_checkpoint(arena: LoRAArena, in_dir: str | Path, layout: Optional[CheckpointLayout] = None) -> list:
    """Load every adapter of the arena from ``in_dir`` (written by :func:`save_checkpoint` under
    any layout): this rank's layers, cut to this rank's tensor-parallel shard.  Returns one
    ``{"step", "data_cursor", "extra"}`` per adapter (``None`` where no training state exists)."""
    layout = layout or CheckpointLayout()
    metas = []

    def cut(tensors):
        return tp_shard(tensors, layout.tp_rank, layout.tp_size)

    for i, spec in enumerate(arena.adapters):
        d = Path(in_dir) / spec.name
        local_spec = arena.adapters[i]
        arena.import_adapter(i, cut(peft_io.read_adapter_tensors(d, arena.layers, local_spec, arena.device)))
        state_file = d / "training_state.pt"
        if state_file.exists() and arena.master is not None:
            metas.append(peft_io.apply_training_state(arena, i, peft_io.read_training_state(state_file), transform=cut))
        else:
            metas.append(None)
    return metas
