"""Public ops: the fused LoRA linear layers, their batch tables, CPU oracles and NF4 weights.

Names follow the reference's public surface (``lorafusion/ops/lora_v1.py:186-200``,
``lorafusion/ops/multi_lora.py:295-453,795-830``, ``lorafusion/ops/lora_torch_ref.py``).
Importing this package does not load the CUDA library; that happens on the first kernel call.
"""

from .batch_info import MultiLoRABatchInfo, prepare_multi_lora_batch_info, single_adapter_batch_info
from .lora import (LoRAStack, fused_linear_lora, fused_linear_multi_lora, lora_linear_backward,
                   lora_linear_forward, set_nf4_fused_max_tokens, set_unfused_baseline)
from .nf4 import NF4Weight, dequantize_nf4, quantize_nf4
from .reference import torch_ref_linear_lora, torch_ref_linear_multi_lora

__all__ = [
    "MultiLoRABatchInfo", "prepare_multi_lora_batch_info", "single_adapter_batch_info", "LoRAStack",
    "fused_linear_lora", "fused_linear_multi_lora", "lora_linear_forward", "lora_linear_backward",
    "set_unfused_baseline", "set_nf4_fused_max_tokens", "NF4Weight", "quantize_nf4", "dequantize_nf4",
    "torch_ref_linear_lora", "torch_ref_linear_multi_lora",
]
