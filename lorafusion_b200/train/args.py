"""Configuration dataclasses and a flag parser for the training / benchmark drivers.

Field names follow the reference's three argument groups so its launch scripts translate one
to one (``lorafusion/train/training_utils.py:94-349``: ``ModelArguments``,
``TrainingArguments``, ``MockDataArguments``, parsed there with ``HfArgumentParser``).  Flags
that selected third-party fast paths in the reference (``use_flash_attn``,
``liger_kernel_level``, ``torch_compile_level``, ``merge_qkv_proj``, ``apply_fused_lora``) are
accepted and ignored: the native kernels are the only path here.  New fields describe what the
reference could not do: ``tensor_parallel_size`` and the gradient-sync implementation.
"""

from __future__ import annotations

import argparse
import dataclasses
from dataclasses import dataclass, field, fields
from typing import Optional, Sequence

from ..models.config import ALL_LINEAR, AdapterSpec


def parse_list(text, cast=float) -> list:
    """``"16 16 32 64"`` or ``"16,16,32,64"`` -> list."""
    if isinstance(text, (list, tuple)):
        return [cast(v) for v in text]
    return [cast(v) for v in str(text).replace(",", " ").split()]


@dataclass
class ModelArguments:
    model_name_or_path: str = "llama-3.1-8b"
    dtype: str = "bfloat16"
    num_layers_for_debugging: Optional[int] = None
    disable_optimizer_for_debugging: bool = False
    lora_alpha: float = 32.0
    lora_dropout: float = 0.1
    lora_r: int = 16
    lora_target_modules: str = "all-linear"
    load_in_4bit: bool = False
    use_nested_quant: bool = True
    bnb_4bit_quant_type: str = "nf4"
    use_multi_lora: bool = False
    num_multi_loras: int = 1
    multi_lora_alpha: str = "32.0"
    multi_lora_dropout_p: str = "0.1"
    multi_lora_r: str = "16"
    # accepted for script compatibility, no effect
    use_flash_attn: bool = True
    liger_kernel_level: str = "disable"
    torch_compile_level: str = "disable"
    merge_qkv_proj: bool = True
    apply_fused_lora: bool = True
    use_torch_optimizer: bool = False

    def adapter_specs(self) -> list:
        targets = ALL_LINEAR if self.lora_target_modules == "all-linear" else tuple(
            parse_list(self.lora_target_modules, str))
        if not self.use_multi_lora:
            return [AdapterSpec("default", self.lora_r, self.lora_alpha, self.lora_dropout, targets)]
        n = self.num_multi_loras

        def expand(text, cast):
            v = parse_list(text, cast)
            if len(v) == 1:
                v = v * n
            if len(v) != n:
                raise ValueError(f"expected 1 or {n} values, got {text!r}")
            return v

        rs, alphas, ps = expand(self.multi_lora_r, int), expand(self.multi_lora_alpha, float), \
            expand(self.multi_lora_dropout_p, float)
        return [AdapterSpec(f"lora_{i}", rs[i], alphas[i], ps[i], targets) for i in range(n)]


@dataclass
class TrainingArguments:
    output_dir: str = "./outputs"
    max_steps: int = 10
    learning_rate: float = 1e-4
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    seed: int = 42
    per_device_train_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    global_batch_size: Optional[int] = None
    use_fsdp: bool = False
    pipeline_parallel_size: int = 1
    tensor_parallel_size: int = 1
    gradient_checkpointing: bool = True
    gradient_checkpointing_layers: Optional[int] = None
    profile: bool = False
    use_timers: bool = False
    multi_lora_max_microbatch_tokens: int = 16384
    multi_lora_global_batch_sizes: str = "8"
    benchmark_baseline_mlora_schedule: bool = False
    grad_sync: str = "auto"            # auto | fused | nccl
    save_adapters: bool = False
    resume_from: Optional[str] = None
    logging_steps: int = 1

    def resolve_batch(self, dp_size: int) -> None:
        """Keep ``global_batch_size = per_device_train_batch_size * dp * grad_accumulation``."""
        if self.global_batch_size is None:
            self.global_batch_size = self.per_device_train_batch_size * dp_size * self.gradient_accumulation_steps
        else:
            denom = self.per_device_train_batch_size * dp_size
            if self.global_batch_size % denom:
                raise ValueError("global_batch_size must be divisible by per-device batch size x dp")
            self.gradient_accumulation_steps = self.global_batch_size // denom

    def recompute_mode(self):
        if not self.gradient_checkpointing:
            return False
        return True if self.gradient_checkpointing_layers is None else "auto"


@dataclass
class MockDataArguments:
    dataset_path: Optional[str] = None           # dataset_distributions.json in the reference layout
    dataset_name: str = "mix"
    dataset_seed: int = 0
    permutation: int = 1
    num_samples: int = 1000
    multi_lora_dataset_schedule_path: Optional[str] = None
    adapter_to_dataset: str = "short medium long xlong"
    use_dummy_fixed_length_dataset: bool = False
    dummy_fixed_length: int = 1024
    max_seq_len: int = 8192


def _add_dataclass(parser: argparse.ArgumentParser, cls) -> None:
    for f in fields(cls):
        default = f.default if f.default is not dataclasses.MISSING else None
        kind = f.type if isinstance(f.type, type) else None
        text = str(f.type)
        if "bool" in text:
            parser.add_argument(f"--{f.name}", type=lambda s: str(s).lower() in ("1", "true", "yes"),
                                default=default, nargs="?", const=True)
        elif "int" in text and "str" not in text:
            parser.add_argument(f"--{f.name}", type=int, default=default)
        elif "float" in text:
            parser.add_argument(f"--{f.name}", type=float, default=default)
        else:
            parser.add_argument(f"--{f.name}", type=str, default=default)
        del kind


def parse_args_into_dataclasses(argv: Optional[Sequence[str]] = None,
                                classes=(ModelArguments, TrainingArguments, MockDataArguments)):
    """``--field value`` flags for every field of the given dataclasses (the role
    ``HfArgumentParser`` plays in ``benchmarks_paper/bench_multi_gpu.py:743-755``)."""
    parser = argparse.ArgumentParser()
    for cls in classes:
        _add_dataclass(parser, cls)
    ns, unknown = parser.parse_known_args(argv)
    if unknown:
        raise SystemExit(f"unknown arguments: {unknown}")
    out = []
    for cls in classes:
        out.append(cls(**{f.name: getattr(ns, f.name) for f in fields(cls)}))
    return tuple(out)
