"""Unfused PyTorch oracles for the fused LoRA linear layers.  They run on CPU in fp32 and
define the semantics every kernel is tested against:

    y  = x W^T + bias + alpha * (dropout(x) A^T) B^T
    dB = alpha * dY^T (dropout(x) A^T)        dA = alpha * (dY B)^T dropout(x)
    dX = dY W + alpha * keep (.) (dY B A) / (1 - p)

(same algebra as ``lorafusion/ops/lora_torch_ref.py:6-120``; the multi-adapter variant
applies dropout to the LoRA branch only, which is what that oracle -- not the reference's
fused multi-LoRA forward -- does).  The dropout mask is the counter-based one of
``ops/philox.py`` so that fused kernels can be compared bit for bit on the mask.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from .philox import keep_mask


def _dropout(x2d: torch.Tensor, p: float, seed: int, stream_id: int, row_offset: int = 0):
    if p <= 0.0:
        return x2d, None
    keep = keep_mask(x2d.shape[0], x2d.shape[1], p, seed, stream_id, row_offset).to(x2d.device)
    xh = torch.where(keep, x2d.float() / (1.0 - p), torch.zeros((), device=x2d.device))
    return xh.to(x2d.dtype), keep


def torch_ref_linear_lora(x: torch.Tensor, linear_w: torch.Tensor, lora_a: torch.Tensor,
                          lora_b: torch.Tensor, alpha: float, dropout_p: float = 0.0,
                          seed: int = 0, stream_id: int = 0,
                          linear_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable unfused LoRA linear.  ``x`` is ``[..., K]``; ``alpha`` is the LoRA
    scaling factor (``lora_alpha / r``)."""
    shape = x.shape
    x2d = x.reshape(-1, shape[-1])
    y = x2d @ linear_w.t()
    if linear_bias is not None:
        y = y + linear_bias
    if dropout_p > 0.0:
        keep = keep_mask(x2d.shape[0], x2d.shape[1], dropout_p, seed, stream_id).to(x.device)
        xh = torch.where(keep, x2d / (1.0 - dropout_p), torch.zeros((), dtype=x.dtype, device=x.device))
    else:
        xh = x2d
    y = y + (xh @ lora_a.t()) @ lora_b.t() * alpha
    return y.reshape(*shape[:-1], linear_w.shape[0])


def torch_ref_linear_multi_lora(padded_x: torch.Tensor, linear_w: torch.Tensor,
                                lora_a_list: Sequence[torch.Tensor],
                                lora_b_list: Sequence[torch.Tensor],
                                seq_len_list: Sequence[int], padded_seq_len_list: Sequence[int],
                                lora_idx_list: Sequence[int], alpha_list: Sequence[float],
                                dropout_p_list: Sequence[float], seed: int = 0, stream_id: int = 0,
                                linear_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable unfused multi-adapter LoRA linear on a packed batch.

    Segment ``i`` occupies ``padded_seq_len_list[i]`` rows and uses adapter
    ``lora_idx_list[i]`` (an index into the A/B lists, ``< 0`` = base model only).  Every row
    of a segment, padding rows included, goes through the adapter: padding rows are
    separate dummy sequences whose outputs are never used and whose gradients are zero.
    """
    shape = padded_x.shape
    x2d = padded_x.reshape(-1, shape[-1])
    y = x2d @ linear_w.t()
    if linear_bias is not None:
        y = y + linear_bias
    pieces = []
    start = 0
    for i, plen in enumerate(padded_seq_len_list):
        seg = x2d[start:start + plen]
        ys = y[start:start + plen]
        a = lora_idx_list[i]
        if a >= 0:
            p = dropout_p_list[i]
            if p > 0.0:
                keep = keep_mask(plen, seg.shape[1], p, seed, stream_id, row_offset=start).to(seg.device)
                xh = torch.where(keep, seg / (1.0 - p), torch.zeros((), dtype=seg.dtype, device=seg.device))
            else:
                xh = seg
            ys = ys + (xh @ lora_a_list[a].t()) @ lora_b_list[a].t() * alpha_list[i]
        pieces.append(ys)
        start += plen
    if start < x2d.shape[0]:
        pieces.append(y[start:])
    return torch.cat(pieces, 0).reshape(*shape[:-1], linear_w.shape[0])
