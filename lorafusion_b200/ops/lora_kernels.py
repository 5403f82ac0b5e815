"""Kernel-level building blocks of the fused (multi-)LoRA linear layer.

Every function here is one launch of the tcgen05 GEMM template with a different operand
layout / epilogue; together they replace the reference's Triton kernels K1-K11 and its
cuBLAS calls for the skinny products (``lorafusion/ops/lora_v1.py:87-166``,
``lorafusion/ops/multi_lora.py:456-600``):

================  =========================================  ===============================
function          computes                                   reference counterpart
================  =========================================  ===============================
``lora_down``     ``S' = alpha_a * drop(X) A_a^T``            dropout.py + ``X̂ @ Aᵀ`` (cuBLAS),
                                                              fused_dropout_matmul.py
``base_lora_fwd`` ``Y = X W^T + S' B_a^T (+ bias)``           fused_(multi_)lora_xw_sb(_tma).py
``lora_ds``       ``dS = alpha_a * dY B_a``                   fused_(multi_)lora_dys_dyb.py (dS half)
``lora_db``       ``dB_a += dY^T S'``                         fused_(multi_)lora_dys_dyb.py (dB half)
``lora_da``       ``dA_a += dS^T drop(X)``                    ``dSᵀ @ X̂`` (cuBLAS loop)
``base_lora_dx``  ``dX = dY W + keep (.) (dS A_a)/(1-p)``     fused_(multi_)lora_dyw_dsa(_tma).py
================  =========================================  ===============================

Conventions
-----------
* Tokens are packed ``[M, features]``; every 128-row tile belongs to one adapter
  (``tile_adapter[m_tile]``, ``-1`` = no adapter) -- the solver pads each adapter's
  segment to a multiple of 128 tokens.
* Adapters are stacked and rank-padded to ``R`` (64, 128, 192 or 256) with zeros:
  ``A_all [n, R, K]``, ``B_all [n, N, R]``; the kernels index them by adapter id, so there
  are no per-call pointer tables and no limit of four adapters.
* ``alpha`` (= lora_alpha / r) is applied to the fp32 accumulator when ``S'`` and ``dS``
  are produced, never folded into bf16 weights.
* The dropout mask is regenerated from Philox (``ops/philox.py``) -- nothing is stored.
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Optional, Sequence

import torch

from . import _native as nv
from .gemm import launch_gemm
from .philox import dropout_threshold

RANK_PAD = 64
RANK_PADS = (64, 128, 192, 256)  # stacked-rank widths the skinny kernels are built for
TILE_M = 128
# N tile of the dX kernel with dropout: 256 = two single-buffered accumulators,
# 128 = two double-buffered accumulators
DROPMIX_BN = int(__import__('os').environ.get('LORAFUSION_B200_DROPMIX_BN', '256'))


@dataclass
class DropoutSpec:
    """Dropout state of one LoRA linear call: a seed, a stream id unique to the call site
    (layer / projection) and either one ``p`` or per-adapter thresholds."""

    seed: int = 0
    stream_id: int = 0
    p: float = 0.0
    adapter_thresh16: Optional[torch.Tensor] = None  # int32/uint32 [n_adapters]
    adapter_inv_keep: Optional[torch.Tensor] = None  # fp32 [n_adapters]
    row_offset: int = 0
    col_offset: int = 0

    @property
    def active(self) -> bool:
        return self.p > 0.0 or self.adapter_thresh16 is not None

    def kwargs(self) -> dict:
        return dict(
            thresh16=dropout_threshold(self.p),
            inv_keep=1.0 / (1.0 - self.p) if self.p > 0 else 1.0,
            adapter_thresh16=self.adapter_thresh16,
            adapter_inv_keep=self.adapter_inv_keep,
            seed=self.seed,
            stream_id=self.stream_id,
            row_offset=self.row_offset,
            col_offset=self.col_offset,
        )


NO_DROPOUT = DropoutSpec()


@dataclass
class SegmentTable:
    """Token segments of one packed microbatch: ``(adapter, start, end)`` with ``start`` and
    ``end`` multiples of 128 and at most one segment per adapter."""

    segments: Sequence[tuple[int, int, int]]
    device: torch.device
    total_rows: Optional[int] = None
    _cache: dict = field(default_factory=dict)

    def split_plan(self, features: int):
        """``(work list, owner)`` with long segments cut into token chunks, or ``None`` when the
        plain work list already fills the GPU.  The work list's fourth column is the CHUNK index
        (the slice of a partial-result buffer the chunk writes); ``owner[chunk]`` = its adapter."""
        key = ("split", features)
        if key not in self._cache:
            self._cache[key] = _split_plan(self, features)
        return self._cache[key]

    def tiles_for(self, features: int) -> torch.Tensor:
        """int32 ``[n_tiles, 4]`` work list ``(feature0, token0, k_blocks, adapter)``."""
        t = self._cache.get(features)
        if t is None:
            rows = []
            seen = set()
            for adapter, start, end in self.segments:
                if adapter < 0 or end <= start:
                    continue
                if adapter in seen:
                    raise ValueError("an adapter may own only one token segment per microbatch")
                seen.add(adapter)
                last = self.total_rows is not None and end >= self.total_rows
                if start % TILE_M or (end % TILE_M and not last):
                    raise ValueError("segment bounds must be multiples of 128 tokens")
                for f0 in range(0, features, TILE_M):
                    rows.append((f0, start, (end - start + 63) // 64, adapter))
            t = torch.tensor(rows, dtype=torch.int32).reshape(-1, 4).to(self.device)
            self._cache[features] = t
        return t


# A gradient kernel gives every (segment, 128-feature tile) to one CTA, which walks all tokens of
# the segment.  With few long segments (one adapter, 8K tokens, 4096 features: 32 work items) most
# SMs idle, so such segments are cut in token chunks that write PARTIAL results, summed afterwards.
_SPLIT_BELOW_ITEMS = 96      # enough work items already: leave the segments whole
_SPLIT_TARGET_ITEMS = 148
_SPLIT_MAX_CHUNKS = 8
_SPLIT_MIN_TOKENS = 1024


def _split_plan(table: SegmentTable, features: int):
    segs = [(a, s0, e0) for a, s0, e0 in table.segments if a >= 0 and e0 > s0]
    f_tiles = (features + TILE_M - 1) // TILE_M
    items = len(segs) * f_tiles
    if not segs or items >= _SPLIT_BELOW_ITEMS:
        return None
    want = min(_SPLIT_MAX_CHUNKS, -(-_SPLIT_TARGET_ITEMS // items))
    rows, owner = [], []
    for a, s0, e0 in segs:
        n_chunks = max(1, min(want, (e0 - s0) // _SPLIT_MIN_TOKENS))
        step = -(-(e0 - s0) // n_chunks)
        step = -(-step // TILE_M) * TILE_M
        for c0 in range(s0, e0, step):
            c1 = min(e0, c0 + step)
            v = len(owner)
            owner.append(a)
            for f0 in range(0, features, TILE_M):
                rows.append((f0, c0, (c1 - c0 + 63) // 64, v))
    if len(owner) == len(segs):
        return None   # nothing was cut
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, 4).to(table.device), owner


def _flat2d(t: torch.Tensor) -> torch.Tensor:
    return t.reshape(-1, t.shape[-1])


def lora_down(x: torch.Tensor, a_all: torch.Tensor, *, tile_adapter: Optional[torch.Tensor],
              adapter_scale: Optional[torch.Tensor], scale: float = 1.0,
              dropout: DropoutSpec = NO_DROPOUT, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``S'[M, R] = alpha_a * dropout(x)[M, K] @ A_a[R, K]^T`` with the adapter of each tile."""
    M, K = x.shape
    n, R, K2 = a_all.shape
    assert K2 == K and R in RANK_PADS
    if out is None:
        out = torch.empty((M, R), dtype=torch.bfloat16, device=x.device)
    launch_gemm(a=x, b=_flat2d(a_all), out=out, M=M, N=R, K=K, bn=R,
                epi=nv.EPI_BF16_ADAPTER_SCALE, mask_a=dropout.active,
                tile_adapter=tile_adapter, b_adapter_rows=R, adapter_scale=adapter_scale,
                scale=scale, **dropout.kwargs())
    return out


def base_lora_fwd(x: torch.Tensor, w: torch.Tensor, s: Optional[torch.Tensor],
                  b_all: Optional[torch.Tensor], *, tile_adapter: Optional[torch.Tensor],
                  bias: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``Y[M, N] = x[M, K] @ w[N, K]^T + S'[M, R] @ B_a[N, R]^T (+ bias)``."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    kw = {}
    if s is not None:
        n, N2, R = b_all.shape
        assert N2 == N and s.shape == (M, R)
        kw = dict(a2=s, b2=_flat2d(b_all), K2=R, b2_adapter_rows=N, tile_adapter=tile_adapter)
    launch_gemm(a=x, b=w, out=out, M=M, N=N, K=K, bn=256 if N >= 256 else 128, bias=bias, tuned="fwd", **kw)
    return out


def lora_ds(dy: torch.Tensor, b_all: torch.Tensor, *, tile_adapter: Optional[torch.Tensor],
            adapter_scale: Optional[torch.Tensor], scale: float = 1.0,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dS[M, R] = alpha_a * dy[M, N] @ B_a[N, R]``."""
    M, N = dy.shape
    n, N2, R = b_all.shape
    assert N2 == N and R in RANK_PADS
    if out is None:
        out = torch.empty((M, R), dtype=torch.bfloat16, device=dy.device)
    launch_gemm(a=dy, b=_flat2d(b_all), out=out, M=M, N=R, K=N, b_mn=True, bn=R,
                epi=nv.EPI_BF16_ADAPTER_SCALE, tile_adapter=tile_adapter, b_adapter_rows=N,
                adapter_scale=adapter_scale, scale=scale)
    return out


def lora_db(dy: torch.Tensor, s: torch.Tensor, segs: SegmentTable, db_all: torch.Tensor) -> None:
    """``dB_all[a][N, R] += dy[seg_a]^T @ S'[seg_a]`` (fp32, one owner CTA per element)."""
    M, N = dy.shape
    n, N2, R = db_all.shape
    assert N2 == N and s.shape == (M, R) and db_all.dtype == torch.float32
    plan = segs.split_plan(N)
    if plan is not None:
        tiles, owner = plan
        tmp = torch.zeros((len(owner), N, R), dtype=torch.float32, device=dy.device)
        launch_gemm(a=dy, b=s, out=tmp, M=N, N=R, K=M, a_mn=True, b_mn=True, bn=R,
                    epi=nv.EPI_F32_ACCUM, seg_tiles=tiles, ldo=R, out_adapter_stride=N * R)
        _fold_chunks(tmp, owner, db_all)
        return
    tiles = segs.tiles_for(N)
    if tiles.shape[0] == 0:
        return
    launch_gemm(a=dy, b=s, out=db_all, M=N, N=R, K=M, a_mn=True, b_mn=True, bn=R,
                epi=nv.EPI_F32_ACCUM, seg_tiles=tiles, ldo=R, out_adapter_stride=N * R)


def lora_da(x: torch.Tensor, ds: torch.Tensor, segs: SegmentTable, da_all: torch.Tensor, *,
            dropout: DropoutSpec = NO_DROPOUT) -> None:
    """``dA_all[a][R, K] += dS[seg_a]^T @ dropout(x)[seg_a]`` (fp32)."""
    M, K = x.shape
    n, R, K2 = da_all.shape
    assert K2 == K and ds.shape == (M, R) and da_all.dtype == torch.float32
    plan = segs.split_plan(K)
    if plan is not None:
        tiles, owner = plan
        drop = dropout
        if dropout.adapter_thresh16 is not None:   # per-adapter rates follow the chunks
            idx = torch.tensor(owner, dtype=torch.long, device=x.device)
            drop = replace(dropout, adapter_thresh16=dropout.adapter_thresh16[idx].contiguous(),
                           adapter_inv_keep=dropout.adapter_inv_keep[idx].contiguous())
        tmp = torch.zeros((len(owner), R, K), dtype=torch.float32, device=x.device)
        launch_gemm(a=x, b=ds, out=tmp, M=K, N=R, K=M, a_mn=True, b_mn=True, bn=R,
                    epi=nv.EPI_F32_ACCUM, mask_a=drop.active, seg_tiles=tiles, ldo=K,
                    out_transposed=True, out_adapter_stride=R * K, **drop.kwargs())
        _fold_chunks(tmp, owner, da_all)
        return
    tiles = segs.tiles_for(K)
    if tiles.shape[0] == 0:
        return
    launch_gemm(a=x, b=ds, out=da_all, M=K, N=R, K=M, a_mn=True, b_mn=True, bn=R,
                epi=nv.EPI_F32_ACCUM, mask_a=dropout.active, seg_tiles=tiles, ldo=K,
                out_transposed=True, out_adapter_stride=R * K, **dropout.kwargs())


def _fold_chunks(tmp: torch.Tensor, owner: Sequence[int], out_all: torch.Tensor) -> None:
    """``out_all[a] += sum of the chunk partials of adapter a``, chunks in token order (a fixed
    order, so the result does not depend on which CTA finished first)."""
    start = 0
    while start < len(owner):
        end = start
        while end < len(owner) and owner[end] == owner[start]:
            end += 1
        out_all[owner[start]] += tmp[start:end].sum(0)
        start = end


def base_lora_dx(dy: torch.Tensor, w: torch.Tensor, ds: Optional[torch.Tensor],
                 a_all: Optional[torch.Tensor], *, tile_adapter: Optional[torch.Tensor],
                 dropout: DropoutSpec = NO_DROPOUT,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dX[M, K] = dy[M, N] @ w[N, K] + keep (.) (dS[M, R] @ A_a[R, K]) / (1 - p)``."""
    M, N = dy.shape
    K = w.shape[1]
    if out is None:
        out = torch.empty((M, K), dtype=torch.bfloat16, device=dy.device)
    kw = {}
    if ds is not None:
        n, R, K2 = a_all.shape
        assert K2 == K and ds.shape == (M, R)
        kw = dict(a2=ds, b2=_flat2d(a_all), K2=R, b2_adapter_rows=R, tile_adapter=tile_adapter)
    if ds is not None and dropout.active:
        launch_gemm(a=dy, b=w, out=out, M=M, N=K, K=N, b_mn=True, b2_mn=True,
                    bn=DROPMIX_BN if K >= 256 else 128, nacc=2,
                    epi=nv.EPI_BF16_DROPMIX, tuned="dx_dropout", **kw, **dropout.kwargs())
    else:
        launch_gemm(a=dy, b=w, out=out, M=M, N=K, K=N, b_mn=True, b2_mn=True,
                    bn=256 if K >= 256 else 128, tuned="dx", **kw)
    return out
