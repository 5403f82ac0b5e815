"""Fused LoRA / multi-LoRA linear layers: functional forward/backward over the sm_100a
kernels, autograd wrappers and the public entry points.

Public API (names and semantics follow the reference so its users can switch):

* ``fused_linear_lora(x, linear_w, lora_a, lora_b, alpha, seed=None, dropout_p=0.0,
  linear_bias=None)`` -- ``lorafusion/ops/lora_v1.py:284-297``
* ``fused_linear_multi_lora(padded_x, linear_w, *, lora_a_list, lora_b_list, ...)`` --
  ``lorafusion/ops/multi_lora.py:762-830``

Differences by design: 2-D and 3-D inputs both work; any number of adapters; the dropout
mask is regenerated, never stored; ``S`` is computed only for each token's own adapter (the
reference multiplies every token by every adapter's ``A``, ``multi_lora.py:502``); dropout
is applied to the LoRA branch (the reference's fused multi-LoRA forward drops the base
branch instead, ``multi_lora.py:502,525-527``); dA/dB are accumulated in fp32 by one owner
CTA per element, so gradients are deterministic (the reference uses fp32 atomics,
``fused_lora_dys_dyb.py:178-179``).

On CPU tensors the entry points evaluate the unfused fp32 oracle of ``ops/reference.py``;
on CUDA tensors they always launch the native kernels.
"""

from __future__ import annotations

import os
import random
from dataclasses import dataclass
from typing import Optional, Sequence, Union

import torch

from . import lora_kernels as lk
from .batch_info import MultiLoRABatchInfo, prepare_multi_lora_batch_info, single_adapter_batch_info
from .nf4 import NF4Weight, dequantize_nf4
from .reference import torch_ref_linear_lora, torch_ref_linear_multi_lora

Weight = Union[torch.Tensor, NF4Weight]


def rank_pad(total_rank: int) -> int:
    """Stacked-rank width the kernels are built for (64, 128, 192 or 256)."""
    for r in lk.RANK_PADS:
        if total_rank <= r:
            return r
    raise ValueError(f"stacked LoRA rank {total_rank} exceeds {lk.RANK_PADS[-1]}")


@dataclass
class LoRAStack:
    """All adapters of one linear layer, stacked and zero-padded to a common rank width:
    ``a [n, R, K]`` / ``b [n, N, R]`` in bf16 (what the kernels read) and optional fp32
    gradient accumulators of the same shapes."""

    a: torch.Tensor
    b: torch.Tensor
    da: Optional[torch.Tensor] = None
    db: Optional[torch.Tensor] = None


# dequantised NF4 weights land in a per-shape scratch buffer reused by every layer
_WEIGHT_SCRATCH: dict[tuple, torch.Tensor] = {}


# Token count up to which an NF4 base weight is expanded inside the GEMM main loop
# (``lf_gemm_nf4``) instead of into scratch memory first.  0 (the default) keeps the fused
# kernel off: on B200 every 128-token tile has to re-expand the weight tile it multiplies and
# the 64 table look-ups + multiplies per row per stage take about 2.6x as long as the stage's
# tcgen05 MMAs, so the kernel ran at ~525 TFLOP/s against ~1400 for dequantise-to-scratch +
# bf16 GEMM at 16384 tokens and was still 1.5x slower at 256 tokens (8192 x 8192 weight;
# ``python -m lorafusion_b200.cli.bench_kernels --nf4-compare``).  One dequantisation pass per
# call costs about 2 % of a 70B training step.
_NF4_FUSED_MAX_TOKENS = int(os.environ.get("LORAFUSION_B200_NF4_FUSED_TOKENS", "0"))


def set_nf4_fused_max_tokens(tokens: int) -> None:
    global _NF4_FUSED_MAX_TOKENS
    _NF4_FUSED_MAX_TOKENS = int(tokens)


def _nf4_fusable(w: "NF4Weight") -> bool:
    return w.packed.is_cuda and w.shape[0] % 256 == 0 and w.shape[1] % 256 == 0


def materialize_weight(w: Weight, tokens: Optional[int] = None) -> Weight:
    """bf16 ``[N, K]`` view of a frozen weight; NF4 weights are expanded into scratch memory
    that the next call with the same shape overwrites (safe under stream ordering) -- unless
    the call is small enough (``tokens``) for the kernel that expands NF4 in its main loop,
    in which case the quantised weight itself is handed on."""
    if isinstance(w, NF4Weight):
        if tokens is not None and tokens <= _NF4_FUSED_MAX_TOKENS and _nf4_fusable(w):
            return w
        key = (w.shape, w.device)
        buf = _WEIGHT_SCRATCH.get(key)
        if buf is None:
            buf = torch.empty(w.shape, dtype=torch.bfloat16, device=w.device)
            _WEIGHT_SCRATCH[key] = buf
        return dequantize_nf4(w, out=buf)
    return w


_UNFUSED = os.environ.get("LORAFUSION_B200_UNFUSED", "0") == "1"


def set_unfused_baseline(enabled: bool) -> None:
    """Switch every LoRA linear of the engine to the unfused baseline (separate base GEMM,
    stored dropout mask, per-adapter cuBLAS GEMMs for the LoRA branch and elementwise adds) --
    the stand-in for the reference's "Torch LoRA" / Megatron-LoRA arm when measuring what the
    fusion buys on the same GPU.  Not used by any default path."""
    global _UNFUSED
    _UNFUSED = bool(enabled)


def _unfused_forward(x, wd, stack, info, stream_id, bias, training):
    y = lk.base_lora_fwd(x, wd, None, None, tile_adapter=None, bias=bias)
    saved = []
    for a, start, end in info.segments:
        if a < 0:
            continue
        p = info.dropout_by_adapter[a] if training else 0.0
        xs = x[start:end]
        xh = torch.nn.functional.dropout(xs, p) if p > 0 else xs
        mask = (xh != 0) if p > 0 else None
        sa_ = xh @ stack.a[a].t()
        y[start:end] += (sa_ @ stack.b[a].t()) * info.alpha_by_adapter[a]
        saved.append((a, start, end, xh, mask, sa_, p))
    return y, saved


def _unfused_backward(dy, x, saved, wd, stack, info, need_dx):
    dx = lk.base_lora_dx(dy, wd, None, None, tile_adapter=None) if need_dx else None
    for a, start, end, xh, mask, sa_, p in saved:
        alpha = info.alpha_by_adapter[a]
        dys = dy[start:end]
        ds = (dys @ stack.b[a]) * alpha
        if stack.db is not None:
            stack.db[a] += (dys.t() @ sa_).float() * alpha
        if stack.da is not None:
            stack.da[a] += (ds.t() @ xh).float()
        if need_dx:
            g = ds @ stack.a[a]
            if mask is not None:
                g = g * mask / (1.0 - p)
            dx[start:end] += g.to(dx.dtype)
    return dx


def lora_linear_forward(x: torch.Tensor, w: Weight, stack: Optional[LoRAStack],
                        info: Optional[MultiLoRABatchInfo], *, stream_id: int = 0,
                        bias: Optional[torch.Tensor] = None, training: bool = True,
                        s: Optional[torch.Tensor] = None):
    """Returns ``(y, s)``; ``s`` (``[M, R]`` bf16) is what the backward needs besides ``x``.
    A precomputed ``s`` (kept from an earlier forward of the same call site) skips the
    down-projection."""
    unfused = _UNFUSED and stack is not None and info is not None
    wd = materialize_weight(w, None if unfused else x.shape[0])
    if unfused:
        return _unfused_forward(x, wd, stack, info, stream_id, bias, training)
    if stack is None or info is None:
        return lk.base_lora_fwd(x, wd, None, None, tile_adapter=None, bias=bias), None
    if s is None or isinstance(s, list):
        drop = info.dropout_spec(stream_id, training)
        s = lk.lora_down(x, stack.a, tile_adapter=info.tile_adapter, adapter_scale=info.adapter_scale,
                         dropout=drop)
    y = lk.base_lora_fwd(x, wd, s, stack.b, tile_adapter=info.tile_adapter, bias=bias)
    return y, s


def lora_linear_backward(dy: torch.Tensor, x: torch.Tensor, s: Optional[torch.Tensor], w: Weight,
                         stack: Optional[LoRAStack], info: Optional[MultiLoRABatchInfo], *,
                         stream_id: int = 0, need_dx: bool = True, training: bool = True):
    """Accumulates dA/dB into ``stack.da`` / ``stack.db`` and returns ``dX`` (or ``None``)."""
    wd = materialize_weight(w, None if isinstance(s, list) else dy.shape[0]) if need_dx else None
    if isinstance(s, list):
        return _unfused_backward(dy, x, s, wd, stack, info, need_dx)
    if stack is None or info is None or s is None:
        return lk.base_lora_dx(dy, wd, None, None, tile_adapter=None) if need_dx else None
    drop = info.dropout_spec(stream_id, training)
    ds = lk.lora_ds(dy, stack.b, tile_adapter=info.tile_adapter, adapter_scale=info.adapter_scale)
    if stack.db is not None:
        lk.lora_db(dy, s, info.segment_table, stack.db)
    if stack.da is not None:
        lk.lora_da(x, ds, info.segment_table, stack.da, dropout=drop)
    if not need_dx:
        return None
    return lk.base_lora_dx(dy, wd, ds, stack.a, tile_adapter=info.tile_adapter, dropout=drop)


class _FusedLoRAFunction(torch.autograd.Function):
    """Autograd node over the functional forward/backward.  ``a_stack`` / ``b_stack`` are the
    padded stacks ``[n, R, K]`` / ``[n, N, R]``; their gradients are returned in their dtype."""

    @staticmethod
    def forward(ctx, x2d, w, bias, a_stack, b_stack, info, stream_id, training):
        stack = LoRAStack(a_stack.detach(), b_stack.detach())
        y, s = lora_linear_forward(x2d, w, stack, info, stream_id=stream_id, bias=bias,
                                   training=training)
        ctx.save_for_backward(x2d, s, a_stack, b_stack)
        ctx.w, ctx.info, ctx.stream_id, ctx.training = w, info, stream_id, training
        return y

    @staticmethod
    def backward(ctx, dy):
        x2d, s, a_stack, b_stack = ctx.saved_tensors
        dy = dy.contiguous()
        need_a, need_b = ctx.needs_input_grad[3], ctx.needs_input_grad[4]
        stack = LoRAStack(
            a_stack.detach(), b_stack.detach(),
            torch.zeros(a_stack.shape, dtype=torch.float32, device=dy.device) if need_a else None,
            torch.zeros(b_stack.shape, dtype=torch.float32, device=dy.device) if need_b else None)
        dx = lora_linear_backward(dy, x2d, s, ctx.w, stack, ctx.info, stream_id=ctx.stream_id,
                                  need_dx=ctx.needs_input_grad[0], training=ctx.training)
        da = stack.da.to(a_stack.dtype) if need_a else None
        db = stack.db.to(b_stack.dtype) if need_b else None
        dbias = dy.float().sum(0).to(dy.dtype) if ctx.needs_input_grad[2] else None
        return dx, None, dbias, da, db, None, None, None


def _pad_stack(a_list: Sequence[Optional[torch.Tensor]], b_list: Sequence[Optional[torch.Tensor]],
               K: int, N: int, device, dtype=torch.bfloat16):
    """Differentiable stacking of per-adapter ``A [r, K]`` / ``B [N, r]`` into padded stacks."""
    ranks = [a.shape[0] for a in a_list if a is not None]
    R = rank_pad(max(ranks) if ranks else 1)
    a_rows, b_rows = [], []
    for a, b in zip(a_list, b_list):
        if a is None:
            a_rows.append(torch.zeros(R, K, dtype=dtype, device=device))
            b_rows.append(torch.zeros(N, R, dtype=dtype, device=device))
        else:
            r = a.shape[0]
            a_rows.append(torch.nn.functional.pad(a.to(dtype), (0, 0, 0, R - r)))
            b_rows.append(torch.nn.functional.pad(b.to(dtype), (0, R - r)))
    return torch.stack(a_rows), torch.stack(b_rows)


def fused_linear_lora(x: torch.Tensor, linear_w: Weight, lora_a: torch.Tensor,
                      lora_b: torch.Tensor, alpha: float, seed: Optional[int] = None,
                      dropout_p: float = 0.0, linear_bias: Optional[torch.Tensor] = None,
                      stream_id: int = 0) -> torch.Tensor:
    """``y = x W^T + bias + alpha * (dropout(x) A^T) B^T`` for ``x [..., K]``, ``W [N, K]``,
    ``A [r, K]``, ``B [N, r]``; ``alpha`` is the LoRA scaling (lora_alpha / r)."""
    if seed is None:
        seed = random.randrange(1 << 31)
    if not x.is_cuda:
        return torch_ref_linear_lora(x, linear_w, lora_a, lora_b, alpha, dropout_p, seed,
                                     stream_id, linear_bias)
    shape = x.shape
    x2d = x.reshape(-1, shape[-1]).contiguous()
    N = lora_b.shape[0]
    a_stack, b_stack = _pad_stack([lora_a], [lora_b], shape[-1], N, x.device)
    info = single_adapter_batch_info(x2d.shape[0], lora_a.shape[0], alpha, dropout_p,
                                     device=x.device, seed=seed)
    y = _FusedLoRAFunction.apply(x2d, linear_w, linear_bias, a_stack, b_stack, info, stream_id,
                                 dropout_p > 0.0)
    return y.reshape(*shape[:-1], N)


def fused_linear_multi_lora(
    padded_x: torch.Tensor,
    linear_w: Weight,
    *,
    lora_a_list: Sequence[Optional[torch.Tensor]],
    lora_b_list: Sequence[Optional[torch.Tensor]],
    batch_info: Optional[MultiLoRABatchInfo] = None,
    seq_len_list: Optional[Sequence[int]] = None,
    padded_seq_len_list: Optional[Sequence[int]] = None,
    lora_idx_list: Optional[Sequence[int]] = None,
    alpha_list: Optional[Sequence[float]] = None,
    dropout_p_list: Optional[Sequence[float]] = None,
    block_to_lookup_table: Optional[torch.Tensor] = None,
    block_to_dropout_p: Optional[torch.Tensor] = None,
    block_to_alpha: Optional[torch.Tensor] = None,
    enable_dropout: bool = True,
    same_dropout_p_value: Optional[float] = None,
    max_r: Optional[int] = None,
    linear_bias: Optional[torch.Tensor] = None,
    seed: int = 0,
    stream_id: int = 0,
) -> torch.Tensor:
    """Multi-adapter fused LoRA linear on a packed batch ``[1, T, K]`` or ``[T, K]``.

    Pass ``batch_info`` (from :func:`prepare_multi_lora_batch_info`), or the per-segment
    lists from which it is built.  ``lora_a_list[i]`` / ``lora_b_list[i]`` belong to adapter
    id ``i`` (``None`` entries are allowed); the reference-style table arguments
    (``block_to_*``, ``max_r``, ``same_dropout_p_value``) are accepted for call
    compatibility and ignored, since the tables live in ``batch_info``.
    """
    del block_to_lookup_table, block_to_dropout_p, block_to_alpha, same_dropout_p_value, max_r
    if batch_info is None:
        if seq_len_list is None:
            raise ValueError("either batch_info or seq_len_list (+ per-segment lists) is required")
        n_seg = len(seq_len_list)
        lora_idx_list = list(range(n_seg)) if lora_idx_list is None else lora_idx_list
        ranks = [lora_a_list[i].shape[0] if i >= 0 and lora_a_list[i] is not None else 0
                 for i in lora_idx_list]
        batch_info = prepare_multi_lora_batch_info(
            seq_len_list, lora_idx_list, ranks, dropout_p_list or [0.0] * n_seg,
            alpha_list or [1.0] * n_seg, device=padded_x.device, seed=seed,
            num_adapters=len(lora_a_list))
    info = batch_info
    if not padded_x.is_cuda:
        return torch_ref_linear_multi_lora(
            padded_x, linear_w, lora_a_list, lora_b_list, info.seq_len_list,
            info.padded_seq_len_list, info.lora_idx_list, info.alpha_list,
            info.dropout_p_list if enable_dropout else [0.0] * len(info.seq_len_list),
            seed=info.seed, stream_id=stream_id, linear_bias=linear_bias)
    shape = padded_x.shape
    x2d = padded_x.reshape(-1, shape[-1]).contiguous()
    N = linear_w.shape[0]
    a_stack, b_stack = _pad_stack(lora_a_list, lora_b_list, shape[-1], N, padded_x.device)
    y = _FusedLoRAFunction.apply(x2d, linear_w, linear_bias, a_stack, b_stack, info, stream_id,
                                 enable_dropout)
    return y.reshape(*shape[:-1], N)
