"""``torch.nn`` modules over the fused LoRA ops, for users who bring their own model.

The reference monkey-patches PEFT's ``LoraLayer.forward`` (``lorafusion/patch/patch_lora.py:44-161``)
and dispatches per call: no manager -> single-adapter op, manager with one active adapter ->
single-adapter op on ``lora_{i}``, otherwise the multi-adapter op.  It also replaces the three
attention projections by one merged ``qkv_proj`` linear
(``lorafusion/patch/patch_transformers.py:165-287``).  Here the same behaviour is offered as
plain modules and two helper functions that rewrite an ``nn.Module`` tree:

* :class:`LoRALinear`       frozen ``nn.Linear`` weight + one adapter, :func:`fused_linear_lora`
* :class:`MultiLoRALinear`  frozen weight + ``n`` adapters named ``lora_{i}``; the packed
  microbatch's :class:`MultiLoRABatchInfo` comes from a :class:`MultiLoRAManager` (newest entry
  in forward, oldest in backward / recomputation) or from ``set_batch_info``
* :func:`apply_lora`        swap every targeted ``nn.Linear`` for one of the above
* :func:`merge_qkv_proj`    fuse sibling ``q_proj`` / ``k_proj`` / ``v_proj`` linears into one

On CPU tensors the ops fall back to the plain-PyTorch oracle, so the modules run anywhere.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
from torch import nn

from .batch_info import MultiLoRABatchInfo
from .lora import fused_linear_lora, fused_linear_multi_lora


def _init_lora_pair(r: int, in_features: int, out_features: int, device, dtype):
    """PEFT's default init: A ~ kaiming-uniform(a = sqrt 5), B = 0."""
    a = torch.empty(r, in_features, device=device, dtype=dtype)
    nn.init.kaiming_uniform_(a, a=math.sqrt(5))
    b = torch.zeros(out_features, r, device=device, dtype=dtype)
    return nn.Parameter(a), nn.Parameter(b)


class LoRALinear(nn.Module):
    """``y = x W^T + bias + (alpha / r) * dropout(x) A^T B^T`` with a frozen ``W``."""

    def __init__(self, base: nn.Linear, r: int = 16, lora_alpha: float = 32.0, lora_dropout: float = 0.1,
                 seed: int = 0, stream_id: int = 0):
        super().__init__()
        self.in_features, self.out_features = base.in_features, base.out_features
        self.weight = nn.Parameter(base.weight.detach(), requires_grad=False)
        self.bias = None if base.bias is None else nn.Parameter(base.bias.detach(), requires_grad=False)
        self.r, self.lora_alpha, self.lora_dropout = r, lora_alpha, lora_dropout
        self.lora_A, self.lora_B = _init_lora_pair(r, self.in_features, self.out_features,
                                                   base.weight.device, base.weight.dtype)
        self.seed, self.stream_id = seed, stream_id
        self._calls = 0

    @property
    def scaling(self) -> float:
        return self.lora_alpha / self.r

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        p = self.lora_dropout if self.training else 0.0
        # a fresh mask per call, reproducible from (seed, call count)
        self._calls += 1
        return fused_linear_lora(x, self.weight, self.lora_A, self.lora_B, self.scaling,
                                 seed=self.seed + self._calls, dropout_p=p, linear_bias=self.bias,
                                 stream_id=self.stream_id)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, r={self.r}, alpha={self.lora_alpha}, p={self.lora_dropout}"


class MultiLoRALinear(nn.Module):
    """Frozen linear with several adapters that share packed microbatches.

    ``adapters`` is a list of ``(r, lora_alpha, lora_dropout)``; adapter ``i`` is stored as
    ``lora_A[f"lora_{i}"]`` / ``lora_B[f"lora_{i}"]`` (the reference's PEFT adapter names)."""

    def __init__(self, base: nn.Linear, adapters: Sequence[tuple], manager=None, stream_id: int = 0):
        super().__init__()
        self.in_features, self.out_features = base.in_features, base.out_features
        self.weight = nn.Parameter(base.weight.detach(), requires_grad=False)
        self.bias = None if base.bias is None else nn.Parameter(base.bias.detach(), requires_grad=False)
        self.adapter_cfgs = [tuple(a) for a in adapters]
        self.lora_A, self.lora_B = nn.ParameterDict(), nn.ParameterDict()
        for i, (r, _, _) in enumerate(self.adapter_cfgs):
            a, b = _init_lora_pair(r, self.in_features, self.out_features, base.weight.device, base.weight.dtype)
            self.lora_A[f"lora_{i}"], self.lora_B[f"lora_{i}"] = a, b
        self.manager = manager
        self.stream_id = stream_id
        self._info: Optional[MultiLoRABatchInfo] = None

    def set_batch_info(self, info: Optional[MultiLoRABatchInfo]) -> None:
        self._info = info

    def _current_info(self) -> Optional[MultiLoRABatchInfo]:
        if self._info is not None:
            return self._info
        if self.manager is None:
            return None
        # forward of a new microbatch reads the newest entry; a recomputation during the
        # backward pass reads the oldest in-flight one
        return self.manager.get_current_batch_info()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        info = self._current_info()
        if info is None:
            raise RuntimeError("MultiLoRALinear needs a MultiLoRABatchInfo (manager or set_batch_info)")
        n = len(self.adapter_cfgs)
        active = sorted({i for i in info.lora_idx_list if i >= 0})
        if len(active) == 1 and len(info.seq_len_list) == 1:
            # one adapter owns the whole microbatch: the single-adapter op is enough
            i = active[0]
            r, alpha, _ = self.adapter_cfgs[i]
            p = info.dropout_p_list[0] if self.training else 0.0
            return fused_linear_lora(x, self.weight, self.lora_A[f"lora_{i}"], self.lora_B[f"lora_{i}"],
                                     alpha / r, seed=info.seed, dropout_p=p, linear_bias=self.bias,
                                     stream_id=self.stream_id)
        return fused_linear_multi_lora(
            x, self.weight,
            lora_a_list=[self.lora_A[f"lora_{i}"] for i in range(n)],
            lora_b_list=[self.lora_B[f"lora_{i}"] for i in range(n)],
            batch_info=info, enable_dropout=self.training, linear_bias=self.bias,
            stream_id=self.stream_id)


ALL_LINEAR_NAMES = ("q_proj", "k_proj", "v_proj", "qkv_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def apply_lora(model: nn.Module, *, r: int = 16, lora_alpha: float = 32.0, lora_dropout: float = 0.1,
               target_modules: Sequence[str] = ALL_LINEAR_NAMES, multi_adapters: Optional[Sequence[tuple]] = None,
               manager=None, seed: int = 0) -> nn.Module:
    """Replace every ``nn.Linear`` whose attribute name is in ``target_modules`` by a
    :class:`LoRALinear` (or :class:`MultiLoRALinear` when ``multi_adapters`` is given), freeze
    everything else, and return ``model``.  Each replaced linear gets its own dropout stream."""
    for prm in model.parameters():
        prm.requires_grad_(False)
    counter = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear) and name in target_modules:
                counter += 1
                if multi_adapters is not None:
                    new = MultiLoRALinear(child, multi_adapters, manager=manager, stream_id=counter)
                else:
                    new = LoRALinear(child, r, lora_alpha, lora_dropout, seed=seed, stream_id=counter)
                setattr(parent, name, new)
    return model


class MergedQKVLinear(nn.Linear):
    """One linear producing ``q | k | v``; remembers the split sizes."""

    def __init__(self, q: nn.Linear, k: nn.Linear, v: nn.Linear):
        has_bias = q.bias is not None
        super().__init__(q.in_features, q.out_features + k.out_features + v.out_features, bias=has_bias,
                         device=q.weight.device, dtype=q.weight.dtype)
        self.split_sizes = (q.out_features, k.out_features, v.out_features)
        with torch.no_grad():
            self.weight.copy_(torch.cat([q.weight, k.weight, v.weight], dim=0))
            if has_bias:
                self.bias.copy_(torch.cat([q.bias, k.bias, v.bias], dim=0))

    def split(self, y: torch.Tensor):
        return torch.split(y, self.split_sizes, dim=-1)

    def to_original(self):
        """Three separate linears with this module's weights (each slice taken from the merged
        tensor with its OWN row offsets)."""
        outs, row = [], 0
        for size in self.split_sizes:
            lin = nn.Linear(self.in_features, size, bias=self.bias is not None, device=self.weight.device,
                            dtype=self.weight.dtype)
            with torch.no_grad():
                lin.weight.copy_(self.weight[row:row + size])
                if self.bias is not None:
                    lin.bias.copy_(self.bias[row:row + size])
            outs.append(lin)
            row += size
        return tuple(outs)


def merge_qkv_proj(model: nn.Module, layer_indices: Optional[Sequence[int]] = None) -> int:
    """Give every module that has ``q_proj``, ``k_proj`` and ``v_proj`` linears a merged
    ``qkv_proj`` (:class:`MergedQKVLinear`) and drop the three originals.  The module's own
    forward must then use ``qkv_proj`` + ``split``.  ``layer_indices`` restricts the rewrite to
    modules whose qualified name contains ``.{index}.`` (the layers of one pipeline stage).
    Returns the number of merged attention blocks."""
    merged = 0
    for qual, mod in list(model.named_modules()):
        if not all(isinstance(getattr(mod, n, None), nn.Linear) for n in ("q_proj", "k_proj", "v_proj")):
            continue
        if layer_indices is not None and not any(f".{i}." in f".{qual}." for i in layer_indices):
            continue
        mod.qkv_proj = MergedQKVLinear(mod.q_proj, mod.k_proj, mod.v_proj)
        del mod.q_proj, mod.k_proj, mod.v_proj
        merged += 1
    return merged
