"""Adapter checkpoints in the PEFT on-disk format, plus per-adapter training state.

The reference never saves anything (its ``SAVE_MODEL`` flag is parsed and ignored,
``benchmarks_paper/scripts/run_single.sh:54,219-221``), but its adapters *are* PEFT LoRA
adapters named ``default`` / ``lora_{i}`` (``lorafusion/train/training_utils.py:604-619``),
so the interchange format is PEFT's: a directory with

* ``adapter_config.json``  (peft_type LORA, r, lora_alpha, lora_dropout, target_modules ...)
* ``adapter_model.safetensors`` with keys
  ``base_model.model.model.layers.{l}.{self_attn|mlp}.{proj}.lora_A.weight`` ``[r, in]`` and
  ``...lora_B.weight`` ``[out, r]``.

Merged projections of this framework (q|k|v, gate|up) are split back into PEFT's per-module
tensors on save and re-merged on load, so checkpoints interoperate with ``PeftModel``.

``save_training_state`` / ``load_training_state`` add what is needed to resume one adapter
independently of the others: fp32 master weights, Adam moments, step count and a data cursor.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch
from safetensors.torch import load_file, save_file

from .adapters import LoRAArena
from .config import AdapterSpec, ModelConfig

_ATTN = {"q_proj", "k_proj", "v_proj", "o_proj"}


def _peft_key(layer: int, module: str, which: str) -> str:
    block = "self_attn" if module in _ATTN else "mlp"
    return f"base_model.model.model.layers.{layer}.{block}.{module}.lora_{which}.weight"


def adapter_config_dict(spec: AdapterSpec, base_model_name: str = "") -> dict:
    return {
        "peft_type": "LORA",
        "task_type": "CAUSAL_LM",
        "base_model_name_or_path": base_model_name,
        "r": spec.r,
        "lora_alpha": spec.lora_alpha,
        "lora_dropout": spec.dropout,
        "target_modules": sorted(spec.target_modules),
        "bias": "none",
        "fan_in_fan_out": False,
        "inference_mode": False,
        "init_lora_weights": True,
        "modules_to_save": None,
        "use_rslora": False,
        "use_dora": False,
    }


def internal_key(layer: int, module: str, which: str) -> str:
    """Key of one LoRA factor in :meth:`LoRAArena.export_adapter` dictionaries."""
    return f"layers.{layer}.{module}.lora_{which}"


def write_adapter_tensors(tensors: dict, spec: AdapterSpec, out_dir: str | Path, *, base_model_name: str = "",
                          dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write a dictionary in :meth:`LoRAArena.export_adapter` form (full, unsharded tensors of
    any set of layers) as a PEFT checkpoint directory."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    peft = {}
    for key, t in tensors.items():
        _, layer, module, which = key.split(".")
        peft[_peft_key(int(layer), module, "A" if which == "lora_A" else "B")] = t.to(dtype).cpu().contiguous()
    save_file(peft, str(out / "adapter_model.safetensors"), metadata={"format": "pt"})
    (out / "adapter_config.json").write_text(json.dumps(adapter_config_dict(spec, base_model_name), indent=2))
    return out


def save_adapter(arena: LoRAArena, adapter: int, out_dir: str | Path, *, base_model_name: str = "",
                 dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write adapter ``adapter`` as a PEFT checkpoint directory.  Single-rank form: under data,
    tensor or pipeline parallelism use :func:`lorafusion_b200.train.checkpoint.save_checkpoint`,
    which first makes the tensors complete."""
    return write_adapter_tensors(arena.export_adapter(adapter), arena.adapters[adapter], out_dir,
                                 base_model_name=base_model_name, dtype=dtype)


def load_adapter_config(in_dir: str | Path, name: Optional[str] = None) -> AdapterSpec:
    cfg = json.loads((Path(in_dir) / "adapter_config.json").read_text())
    return AdapterSpec(name or Path(in_dir).name, r=int(cfg["r"]), lora_alpha=float(cfg["lora_alpha"]),
                       dropout=float(cfg.get("lora_dropout", 0.0)), target_modules=tuple(cfg["target_modules"]))


def read_adapter_tensors(in_dir: str | Path, layers, have: AdapterSpec, device="cpu") -> dict:
    """Read the LoRA factors of ``layers`` from a PEFT checkpoint directory into a dictionary in
    :meth:`LoRAArena.export_adapter` form (fp32, full tensors).  Rank and target modules must
    match ``have``."""
    spec = load_adapter_config(in_dir)
    if spec.r != have.r or set(spec.target_modules) != set(have.target_modules):
        raise ValueError(f"checkpoint (r={spec.r}, targets={sorted(spec.target_modules)}) does not match "
                         f"the adapter slot (r={have.r}, targets={sorted(have.target_modules)})")
    raw = load_file(str(Path(in_dir) / "adapter_model.safetensors"))
    tensors = {}
    for l in layers:
        for module in have.target_modules:
            for which in ("A", "B"):
                k = _peft_key(l, module, which)
                # PEFT writes "...lora_A.weight"; some versions insert the adapter name
                alt = k.replace(f".lora_{which}.weight", f".lora_{which}.default.weight")
                src = raw.get(k, raw.get(alt))
                if src is None:
                    raise KeyError(f"{k} missing from checkpoint")
                tensors[internal_key(l, module, which)] = src.to(device, torch.float32)
    return tensors


def load_adapter(arena: LoRAArena, adapter: int, in_dir: str | Path) -> None:
    """Load a PEFT checkpoint into slot ``adapter`` of the arena (rank and targets must match
    the slot's :class:`AdapterSpec`; only the arena's layers are read, so a pipeline stage
    loads its part of a whole-model checkpoint)."""
    arena.import_adapter(adapter, read_adapter_tensors(in_dir, arena.layers, arena.adapters[adapter], arena.device))


def write_training_state(state: dict, path: str | Path, *, step: int, data_cursor: int = 0,
                         extra: Optional[dict] = None) -> None:
    """``state = {"master" | "m" | "v": {key: full fp32 tensor}}`` with keys as in
    :meth:`LoRAArena.export_adapter`: a layout-independent file, so a run may resume under
    another dp x pp x tp layout than the one that saved it."""
    payload = {"version": 2, "step": int(step), "data_cursor": int(data_cursor), "extra": extra or {},
               "state": {name: {k: t.detach().cpu().clone() for k, t in tensors.items()}
                         for name, tensors in state.items()}}
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    torch.save(payload, str(path))


def read_training_state(path: str | Path) -> dict:
    return torch.load(str(path), map_location="cpu", weights_only=False)


def save_training_state(arena: LoRAArena, adapter: int, path: str | Path, *, data_cursor: int = 0,
                        extra: Optional[dict] = None) -> None:
    """fp32 master / Adam moments of one adapter, keyed by layer and module, plus step count and
    data cursor.  Single-rank form (see :func:`save_adapter`)."""
    write_training_state({name: arena.export_adapter(adapter, name) for name in ("master", "m", "v")}, path,
                         step=arena.steps[adapter], data_cursor=data_cursor, extra=extra)


def apply_training_state(arena: LoRAArena, adapter: int, payload: dict, transform=None) -> dict:
    """Put a payload of :func:`read_training_state` into the arena.  ``transform(tensors) ->
    tensors`` cuts full tensors down to this rank's shard (tensor parallelism); tensors of
    layers the arena does not hold are ignored."""
    if int(payload.get("version", 1)) < 2:  # flat dense ranges of an unsharded single-rank arena
        lo, hi = arena.state_range[adapter]
        if int(payload["numel"]) != hi - lo:
            raise ValueError(f"checkpoint holds {payload['numel']} optimizer elements, adapter {adapter} has {hi - lo}")
        arena.master[lo:hi].copy_(payload["master"])
        arena.m[lo:hi].copy_(payload["m"])
        arena.v[lo:hi].copy_(payload["v"])
        arena.import_adapter(adapter, arena.export_adapter(adapter, "master"))
    else:
        for name, target in (("master", "weights"), ("m", "m"), ("v", "v")):
            tensors = {k: t.to(arena.device) for k, t in payload["state"][name].items()
                       if int(k.split(".")[1]) in set(arena.layers)}
            if transform is not None:
                tensors = transform(tensors)
            arena.import_adapter(adapter, tensors, target=target)  # "weights" also refreshes the bf16 copy
    arena.steps[adapter] = int(payload["step"])
    return {"step": payload["step"], "data_cursor": payload["data_cursor"], "extra": payload["extra"]}


def load_training_state(arena: LoRAArena, adapter: int, path: str | Path) -> dict:
    return apply_training_state(arena, adapter, read_training_state(path))
