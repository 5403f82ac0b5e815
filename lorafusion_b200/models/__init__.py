"""Models: decoder configurations (Llama-3.1-8B / 70B, Qwen2.5-32B shapes), the manually
differentiated decoder stage and its tensor-parallel variant, the adapter arenas, activation
offloading and PEFT-format adapter checkpoints."""

from .adapters import LoRAArena, projection_layout
from .config import ALL_LINEAR, AdapterSpec, ModelConfig, get_model_config

__all__ = ["LoRAArena", "projection_layout", "ALL_LINEAR", "AdapterSpec", "ModelConfig", "get_model_config"]
