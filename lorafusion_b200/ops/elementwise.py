"""Launchers for the memory-bound decoder kernels (``csrc/elementwise``): RMSNorm with fused
residual add, in-place rotary embedding, SwiGLU, embedding gather, chunked cross-entropy and
the multi-tensor Adam step.  All activations are bf16 ``[tokens, features]``."""

from __future__ import annotations

from typing import Optional

import torch

from . import _native as nv


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, res: Optional[torch.Tensor] = None,
                want_rstd: bool = True, out: Optional[torch.Tensor] = None):
    """``h = x (+ res); y = h * rsqrt(mean(h^2) + eps) * w``.  Returns ``(y, h, rstd)``;
    ``h`` is ``x`` itself when there is no residual.  ``out`` (contiguous ``[M, H]``) receives
    ``y`` in place, e.g. this rank's rows of an all-gather buffer."""
    M, H = x.shape
    y = torch.empty_like(x) if out is None else out
    h = torch.empty_like(x) if res is not None else x
    rstd = torch.empty(M, dtype=torch.float32, device=x.device) if want_rstd else None
    nv.call("lf_rmsnorm_fwd", x.data_ptr(), _p(res), w.data_ptr(), y.data_ptr(),
            h.data_ptr() if res is not None else None, _p(rstd), M, H, eps,
            nv.current_stream_ptr())
    return y, h, rstd


def rmsnorm_bwd(dy: torch.Tensor, h: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                dres: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gradient w.r.t. the normalised input (the frozen weight gets none), plus ``dres``."""
    M, H = h.shape
    dx = torch.empty_like(h)
    nv.call("lf_rmsnorm_bwd", dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _p(dres),
            dx.data_ptr(), M, H, nv.current_stream_ptr())
    return dx


def rope_inplace(qkv: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 n_rot_heads: int, head_dim: int, backward: bool = False) -> None:
    """Rotate the first ``n_rot_heads`` heads (q then k) of the packed projection in place."""
    M = qkv.shape[0]
    nv.call("lf_rope_inplace", qkv.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), M,
            n_rot_heads, head_dim, qkv.stride(0), int(backward), nv.current_stream_ptr())


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    M, I2 = gu.shape
    out = torch.empty((M, I2 // 2), dtype=gu.dtype, device=gu.device)
    nv.call("lf_swiglu_fwd", gu.data_ptr(), out.data_ptr(), M, I2 // 2, nv.current_stream_ptr())
    return out


def swiglu_bwd(dout: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    M, I2 = gu.shape
    dgu = torch.empty_like(gu)
    nv.call("lf_swiglu_bwd", dout.data_ptr(), gu.data_ptr(), dgu.data_ptr(), M, I2 // 2,
            nv.current_stream_ptr())
    return dgu


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    M = ids.numel()
    V, H = table.shape
    out = torch.empty((M, H), dtype=table.dtype, device=table.device)
    nv.call("lf_embedding", ids.data_ptr(), table.data_ptr(), out.data_ptr(), M, H, V,
            nv.current_stream_ptr())
    return out


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(a)
    nv.call("lf_add", a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(),
            nv.current_stream_ptr())
    return out


def cross_entropy_inplace(logits: torch.Tensor, labels: torch.Tensor, grad_scale: float,
                          loss_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-token loss of a logits chunk; ``logits`` is overwritten with
    ``grad_scale * d loss / d logits``.  ``labels < 0`` are ignored."""
    M, V = logits.shape
    if loss_out is None:
        loss_out = torch.empty(M, dtype=torch.float32, device=logits.device)
    nv.call("lf_cross_entropy", logits.data_ptr(), labels.data_ptr(), loss_out.data_ptr(), M, V,
            logits.stride(0), grad_scale, nv.current_stream_ptr())
    return loss_out


ADAM_WORK_UNIT = 32768  # elements per CTA (a multiple of 4)


def dp_slice(total: int, rank: int, world: int) -> tuple[int, int]:
    """Element range ``[lo, hi)`` of a region of ``total`` elements that data-parallel rank
    ``rank`` of ``world`` reduces, updates and owns the optimizer state of: regions are cut in
    ``world`` slices of whole 4-element groups."""
    total4 = total // 4
    per = (total4 + world - 1) // world
    return 4 * min(total4, per * rank), 4 * min(total4, per * (rank + 1))


def build_adam_work_items(chunk_rows, *, rank: int = 0, world: int = 1, unit: int = ADAM_WORK_UNIT) -> torch.Tensor:
    """Cut every region of a chunk table (rows ``offset, rows, ld, col0, cols, state``) into
    pieces of at most ``unit`` elements: int32 ``[n, 3]`` rows ``(chunk index, first element,
    element count)`` on the CPU.  With ``world > 1`` only slice ``rank`` of every region is
    covered (slices are whole 4-element groups, the split the fused data-parallel kernel
    uses).  Regions differ in size by two orders of magnitude; equal pieces keep the CTAs of the
    optimizer kernels balanced."""
    items = []
    for ci, row in enumerate(chunk_rows):
        total = int(row[1]) * int(row[2])
        vec = all(int(v) % 4 == 0 for v in (row[0], row[2], row[3], row[4], row[5]))
        if world > 1:
            if not vec:
                raise ValueError("data-parallel slicing needs regions made of whole 4-element groups")
            lo, hi = dp_slice(total, rank, world)
        else:
            lo, hi = 0, total
        step = unit if vec else max(1, unit // 4)
        for first in range(lo, hi, step):
            items.append((ci, first, min(step, hi - first)))
    return torch.tensor(items, dtype=torch.int32).view(-1, 3)


def adam_chunks(chunks: torch.Tensor, grad: torch.Tensor, master: torch.Tensor, m: torch.Tensor,
                v: torch.Tensor, work: torch.Tensor, *, lr: float, beta1: float, beta2: float,
                eps: float, weight_decay: float, step: int, grad_scale: float = 1.0,
                items: Optional[torch.Tensor] = None) -> None:
    """AdamW over the regions listed in ``chunks`` (int64 ``[n, 6]``: offset, rows, ld, col0,
    cols, state).  ``grad`` and ``work`` are addressed by ``offset`` (padded layout), ``master`` /
    ``m`` / ``v`` by ``state`` (dense over the trainable window); consumes and clears the gradient."""
    if chunks.dim() != 2 or chunks.shape[1] != 6:
        raise ValueError("chunk table must be int64 [n, 6]")
    if items is None:  # callers on a hot path pass a cached table (this reads the chunks back)
        items = build_adam_work_items(chunks.cpu().tolist()).to(chunks.device)
    nv.call("lf_adam_chunks", chunks.data_ptr(), items.data_ptr(), items.shape[0], grad.data_ptr(),
            master.data_ptr(), m.data_ptr(), v.data_ptr(), work.data_ptr(), lr, beta1, beta2, eps,
            weight_decay, step, grad_scale, nv.current_stream_ptr())
