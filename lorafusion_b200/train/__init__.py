"""Training front end: argument groups, synthetic data and providers, the multi-LoRA manager,
the single-stage trainer and the dp x pp x tp engine."""

from .args import MockDataArguments, ModelArguments, TrainingArguments, parse_args_into_dataclasses
from .data import LengthDistribution, MicroBatchSpec, MockDataset, NAMED_DISTRIBUTIONS
from .manager import MultiLoRAManager, get_multi_lora_manager, init_multi_lora_manager, reset_multi_lora_manager

__all__ = [
    "MockDataArguments", "ModelArguments", "TrainingArguments", "parse_args_into_dataclasses", "LengthDistribution",
    "MicroBatchSpec", "MockDataset", "NAMED_DISTRIBUTIONS", "MultiLoRAManager", "get_multi_lora_manager",
    "init_multi_lora_manager", "reset_multi_lora_manager",
]
