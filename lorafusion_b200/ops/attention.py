"""Causal variable-length grouped-query attention (head_dim 128) on packed sequences.

Forward and backward run the tcgen05 kernels of ``csrc/attention``; the autograd function
reads q/k/v straight from the packed, already rotated QKV projection ``[tokens, (Hq + 2
Hkv) * 128]`` and returns the gradient in the same packed layout.  This takes the place of
the FlashAttention-2 varlen call the reference reaches through HF's attention interface
(``lorafusion/patch/patch_transformers.py:150-159``; ``cu_seq_lens`` built in
``lorafusion/utils/hf.py:97-103``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _native as nv

HEAD_DIM = 128
TILE = 128


@dataclass
class AttnTiles:
    """128-row work items of a packed batch: int32 ``[n, 4]`` rows
    ``(row0, rows, seq_row0, seq_rows)``, longest key range first."""

    tiles: torch.Tensor
    num_tiles: int


def build_attn_tiles(cu_seqlens, device) -> AttnTiles:
    """Cut every sequence (``cu_seqlens`` = cumulative lengths, host ints) into 128-row
    tiles.  Tiles with the most key rows come first so the longest CTAs start earliest."""
    rows = []
    cs = [int(v) for v in cu_seqlens]
    for b in range(len(cs) - 1):
        start, length = cs[b], cs[b + 1] - cs[b]
        for t0 in range(0, length, TILE):
            rows.append((start + t0, min(TILE, length - t0), start, length))
    rows.sort(key=lambda r: -(r[0] - r[2]))
    t = torch.tensor(rows, dtype=torch.int32).reshape(-1, 4)
    return AttnTiles(t.to(device), len(rows))


def attention_reference(q, k, v, cu_seqlens, scale=None):
    """fp32 PyTorch oracle: q ``[M, Hq, D]``, k/v ``[M, Hkv, D]``; causal within sequences."""
    M, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.zeros(M, Hq, D, dtype=torch.float32, device=q.device)
    cs = [int(x) for x in cu_seqlens]
    for b in range(len(cs) - 1):
        s, e = cs[b], cs[b + 1]
        if e == s:
            continue
        qb = q[s:e].float().transpose(0, 1)
        kb = k[s:e].float().transpose(0, 1).repeat_interleave(Hq // Hkv, dim=0)
        vb = v[s:e].float().transpose(0, 1).repeat_interleave(Hq // Hkv, dim=0)
        sc = (qb @ kb.transpose(1, 2)) * scale
        mask = torch.ones(e - s, e - s, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        out[s:e] = (sc.softmax(-1) @ vb).transpose(0, 1)
    return out


def attention_forward(qkv: torch.Tensor, tiles: AttnTiles, n_q_heads: int, n_kv_heads: int,
                      scale: float | None = None):
    """Functional forward: returns ``(out [T, Hq*128] bf16, lse [Hq, T] fp32)``."""
    M = qkv.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(HEAD_DIM)
    out = torch.empty((M, n_q_heads * HEAD_DIM), dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty((n_q_heads, M), dtype=torch.float32, device=qkv.device)
    k0 = n_q_heads * HEAD_DIM
    v0 = k0 + n_kv_heads * HEAD_DIM
    nv.call("lf_attn_fwd", qkv.data_ptr(), M, qkv.stride(0), 0, k0, v0, n_q_heads, n_kv_heads,
            tiles.tiles.data_ptr(), tiles.num_tiles, out.data_ptr(), out.stride(0),
            lse.data_ptr(), scale, nv.err_word(qkv.device).data_ptr(), nv.current_stream_ptr())
    return out, lse


def attention_backward(qkv: torch.Tensor, out: torch.Tensor, d_out: torch.Tensor, lse: torch.Tensor,
                       tiles: AttnTiles, n_q_heads: int, n_kv_heads: int,
                       scale: float | None = None) -> torch.Tensor:
    """Functional backward: gradient w.r.t. the packed (rotated) QKV, same layout as ``qkv``."""
    M = qkv.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(HEAD_DIM)
    d_out = d_out.contiguous()
    dqkv = torch.empty_like(qkv)
    delta = torch.empty_like(lse)
    k0 = n_q_heads * HEAD_DIM
    v0 = k0 + n_kv_heads * HEAD_DIM
    nv.call("lf_attn_bwd", qkv.data_ptr(), out.data_ptr(), d_out.data_ptr(), dqkv.data_ptr(), M,
            qkv.stride(0), 0, k0, v0, n_q_heads, n_kv_heads, tiles.tiles.data_ptr(), tiles.num_tiles,
            out.stride(0), lse.data_ptr(), delta.data_ptr(), scale,
            nv.err_word(qkv.device).data_ptr(), nv.current_stream_ptr())
    return dqkv


class _PackedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, tiles: AttnTiles, n_q_heads: int, n_kv_heads: int, scale: float):
        out, lse = attention_forward(qkv, tiles, n_q_heads, n_kv_heads, scale)
        ctx.save_for_backward(qkv, out, lse)
        ctx.tiles, ctx.hq, ctx.hkv, ctx.scale = tiles, n_q_heads, n_kv_heads, scale
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, out, lse = ctx.saved_tensors
        dqkv = attention_backward(qkv, out, d_out, lse, ctx.tiles, ctx.hq, ctx.hkv, ctx.scale)
        return dqkv, None, None, None, None


def packed_attention(qkv: torch.Tensor, tiles: AttnTiles, n_q_heads: int, n_kv_heads: int,
                     scale: float | None = None) -> torch.Tensor:
    """``softmax(q k^T * scale, causal) v`` per sequence; returns ``[tokens, Hq * 128]``."""
    if qkv.shape[1] != (n_q_heads + 2 * n_kv_heads) * HEAD_DIM:
        raise ValueError("packed QKV width does not match the head counts (head_dim is 128)")
    scale = scale if scale is not None else 1.0 / math.sqrt(HEAD_DIM)
    return _PackedAttention.apply(qkv, tiles, n_q_heads, n_kv_heads, scale)
