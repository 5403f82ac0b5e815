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


def save_adapter(arena: LoRAArena, adapter: int, out_dir: str | Path, *, base_model_name: str = "",
                 dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write adapter ``adapter`` as a PEFT checkpoint directory."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    spec = arena.adapters[adapter]
    tensors = {}
    for key, t in arena.export_adapter(adapter).items():
        _, layer, module, which = key.split(".")
        tensors[_peft_key(int(layer), module, "A" if which == "lora_A" else "B")] = t.to(dtype).cpu().contiguous()
    save_file(tensors, str(out / "adapter_model.safetensors"), metadata={"format": "pt"})
    (out / "adapter_config.json").write_text(json.dumps(adapter_config_dict(spec, base_model_name), indent=2))
    return out


def load_adapter_config(in_dir: str | Path, name: Optional[str] = None) -> AdapterSpec:
    cfg = json.loads((Path(in_dir) / "adapter_config.json").read_text())
    return AdapterSpec(name or Path(in_dir).name, r=int(cfg["r"]), lora_alpha=float(cfg["lora_alpha"]),
                       dropout=float(cfg.get("lora_dropout", 0.0)), target_modules=tuple(cfg["target_modules"]))


def load_adapter(arena: LoRAArena, adapter: int, in_dir: str | Path) -> None:
    """Load a PEFT checkpoint into slot ``adapter`` of the arena (rank and targets must match
    the slot's :class:`AdapterSpec`)."""
    spec = load_adapter_config(in_dir)
    have = arena.adapters[adapter]
    if spec.r != have.r or set(spec.target_modules) != set(have.target_modules):
        raise ValueError(f"checkpoint (r={spec.r}, targets={sorted(spec.target_modules)}) does not match "
                         f"adapter slot {adapter} (r={have.r}, targets={sorted(have.target_modules)})")
    raw = load_file(str(Path(in_dir) / "adapter_model.safetensors"))
    tensors = {}
    for l in arena.layers:
        for module in have.target_modules:
            for which in ("A", "B"):
                k = _peft_key(l, module, which)
                # PEFT writes "...lora_A.weight"; some versions insert the adapter name
                alt = k.replace(f".lora_{which}.weight", f".lora_{which}.default.weight")
                src = raw.get(k, raw.get(alt))
                if src is None:
                    raise KeyError(f"{k} missing from checkpoint")
                tensors[f"layers.{l}.{module}.lora_{which}"] = src.to(arena.device, torch.float32)
    arena.import_adapter(adapter, tensors)


def save_training_state(arena: LoRAArena, adapter: int, path: str | Path, *, data_cursor: int = 0,
                        extra: Optional[dict] = None) -> None:
    """fp32 master / Adam moments of one adapter (its dense optimizer-state range), step
    count and data cursor."""
    lo, hi = arena.state_range[adapter]
    state = {"step": arena.steps[adapter], "data_cursor": data_cursor, "extra": extra or {},
             "numel": hi - lo,
             "master": arena.master[lo:hi].cpu().clone(),
             "m": arena.m[lo:hi].cpu().clone(),
             "v": arena.v[lo:hi].cpu().clone()}
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    torch.save(state, str(path))


def load_training_state(arena: LoRAArena, adapter: int, path: str | Path) -> dict:
    state = torch.load(str(path), map_location="cpu", weights_only=False)
    lo, hi = arena.state_range[adapter]
    if int(state["numel"]) != hi - lo:
        raise ValueError(f"checkpoint holds {state['numel']} optimizer elements, adapter {adapter} has {hi - lo}")
    arena.master[lo:hi].copy_(state["master"])
    arena.m[lo:hi].copy_(state["m"])
    arena.v[lo:hi].copy_(state["v"])
    # the bf16 working copy follows the restored master weights
    arena.import_adapter(adapter, arena.export_adapter(adapter))
    arena.steps[adapter] = int(state["step"])
    return {"step": state["step"], "data_cursor": state["data_cursor"], "extra": state["extra"]}
