"""CPU implementation of the counter-based dropout mask used by the CUDA kernels.

The mask is a pure function of ``(seed, stream, row, col)``: one Philox4x32-7 call with key
``(seed_lo, seed_hi)`` and counter ``(row, col // 8, stream, 0)`` yields eight 16-bit lanes;
element ``(row, col)`` is kept iff lane ``col % 8`` is ``>= round(p * 65536)``.  This file and
``csrc/common/philox.cuh`` must agree bit for bit -- the GPU tests compare kernels that
regenerate the mask on the fly against oracles that use this one.

The reference stores a Philox-7 mask as a bool tensor and re-reads it
(``lorafusion/ops/triton_ops/dropout.py:18-93``); here it is never materialised on the GPU.
"""

from __future__ import annotations

import numpy as np
import torch

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32(c0, c1, c2, c3, k0: int, k1: int, rounds: int = 7):
    """Vectorised Philox4x32; counters are uint32 arrays of one shape."""
    c0 = c0.astype(np.uint64)
    c1 = c1.astype(np.uint64)
    c2 = c2.astype(np.uint64)
    c3 = c3.astype(np.uint64)
    k0 &= 0xFFFFFFFF
    k1 &= 0xFFFFFFFF
    for _ in range(rounds):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK32
        n0 = hi1 ^ c1 ^ np.uint64(k0)
        n2 = hi0 ^ c3 ^ np.uint64(k1)
        c0, c1, c2, c3 = n0, lo1, n2, lo0
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return (c0.astype(np.uint32), c1.astype(np.uint32), c2.astype(np.uint32),
            c3.astype(np.uint32))


def dropout_threshold(p: float) -> int:
    """16-bit keep threshold for drop probability ``p`` (0 disables dropout)."""
    if p <= 0.0:
        return 0
    if p >= 1.0:
        raise ValueError("dropout p must be < 1")
    return int(round(p * 65536.0))


def keep_mask(rows: int, cols: int, p: float, seed: int, stream: int = 0,
              row_offset: int = 0, col_offset: int = 0) -> torch.Tensor:
    """Boolean keep mask ``[rows, cols]`` identical to the one the kernels regenerate."""
    if p <= 0.0:
        return torch.ones(rows, cols, dtype=torch.bool)
    if col_offset % 8 != 0:
        raise ValueError("col_offset must be a multiple of 8")
    thresh = dropout_threshold(p)
    ncol8 = (cols + 7) // 8
    r = (np.arange(rows, dtype=np.uint32) + np.uint32(row_offset))[:, None]
    c8 = (np.arange(ncol8, dtype=np.uint32) + np.uint32(col_offset // 8))[None, :]
    r, c8 = np.broadcast_arrays(r, c8)
    s = np.full(r.shape, stream & 0xFFFFFFFF, dtype=np.uint32)
    z = np.zeros(r.shape, dtype=np.uint32)
    out = philox4x32(r, c8, s, z, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    lanes = np.empty(r.shape + (8,), dtype=np.uint32)
    for j in range(8):
        lanes[..., j] = (out[j >> 1] >> np.uint32(16 * (j & 1))) & np.uint32(0xFFFF)
    keep = (lanes >= np.uint32(thresh)).reshape(rows, ncol8 * 8)[:, :cols]
    return torch.from_numpy(np.ascontiguousarray(keep))


def apply_dropout(x: torch.Tensor, p: float, seed: int, stream: int = 0, row_offset: int = 0,
                  col_offset: int = 0) -> torch.Tensor:
    """``keep * x / (1 - p)`` computed in fp32 and rounded back to ``x.dtype``, as the
    in-shared-memory masking step of the kernels does."""
    if p <= 0.0:
        return x
    keep = keep_mask(x.shape[0], x.shape[1], p, seed, stream, row_offset, col_offset).to(x.device)
    inv = 1.0 / (1.0 - p)
    return torch.where(keep, x.float() * inv, torch.zeros((), dtype=torch.float32,
                                                           device=x.device)).to(x.dtype)
