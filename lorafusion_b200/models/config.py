"""Decoder architecture descriptions (Llama-3.x and Qwen2.5 shapes) and LoRA adapter specs.

The reference loads HF checkpoints by name (``lorafusion/train/training_utils.py:533-629``);
this framework owns its decoder, so an architecture is a plain dataclass.  The presets carry
the shapes of the three models the reference benchmarks (8B / 32B / 70B) plus miniatures used
by the tests.  head_dim is 128 for every preset (the attention kernels are built for it).
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Optional, Sequence


@dataclass(frozen=True)
class RopeScaling:
    """Llama-3.1 frequency-dependent RoPE scaling."""

    factor: float = 8.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192


@dataclass(frozen=True)
class ModelConfig:
    name: str
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float = 500000.0
    rope_scaling: Optional[RopeScaling] = None
    rms_eps: float = 1e-5
    qkv_bias: bool = False
    head_dim: int = 128
    max_position: int = 8192

    def __post_init__(self):
        if self.head_dim != 128:
            raise ValueError("head_dim must be 128")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def qkv_size(self) -> int:
        return self.q_size + 2 * self.kv_size

    def layer_param_count(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        return h * self.qkv_size + self.q_size * h + 3 * h * i + 2 * h

    def param_count(self) -> int:
        return self.num_layers * self.layer_param_count() + 2 * self.vocab_size * self.hidden_size + self.hidden_size

    def with_layers(self, n: int) -> "ModelConfig":
        return replace(self, num_layers=n, name=f"{self.name}-{n}L")


_LLAMA3_SCALING = RopeScaling()

PRESETS: dict[str, ModelConfig] = {
    "llama-3.1-8b": ModelConfig("llama-3.1-8b", 4096, 32, 32, 8, 14336, 128256, 500000.0, _LLAMA3_SCALING),
    "llama-3.1-70b": ModelConfig("llama-3.1-70b", 8192, 80, 64, 8, 28672, 128256, 500000.0, _LLAMA3_SCALING),
    "qwen2.5-32b": ModelConfig("qwen2.5-32b", 5120, 64, 40, 8, 27648, 152064, 1000000.0, None, 1e-6, True),
    # miniatures for tests and smoke runs
    "tiny": ModelConfig("tiny", 512, 2, 4, 2, 1024, 1024, 10000.0, None),
    "tiny-qwen": ModelConfig("tiny-qwen", 512, 2, 4, 2, 1024, 1024, 10000.0, None, 1e-6, True),
    "small": ModelConfig("small", 1024, 4, 8, 2, 3072, 32000, 500000.0, _LLAMA3_SCALING),
}

ALIASES = {
    "meta-llama/Llama-3.1-8B-Instruct": "llama-3.1-8b",
    "meta-llama/Llama-3.1-70B-Instruct": "llama-3.1-70b",
    "Qwen/Qwen2.5-32B-Instruct": "qwen2.5-32b",
    "8b": "llama-3.1-8b",
    "32b": "qwen2.5-32b",
    "70b": "llama-3.1-70b",
}


def get_model_config(name: str) -> ModelConfig:
    key = ALIASES.get(name, name)
    if key not in PRESETS:
        raise KeyError(f"unknown model '{name}'; known: {sorted(PRESETS)}")
    return PRESETS[key]


ALL_LINEAR = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


@dataclass(frozen=True)
class AdapterSpec:
    """One LoRA adapter (one fine-tuning job): rank, ``lora_alpha`` (scaling = alpha / r),
    dropout and the projections it is attached to."""

    name: str
    r: int = 16
    lora_alpha: float = 32.0
    dropout: float = 0.0
    target_modules: Sequence[str] = field(default_factory=lambda: ALL_LINEAR)

    @property
    def scaling(self) -> float:
        return self.lora_alpha / self.r
