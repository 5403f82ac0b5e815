"""Python launchers for the tcgen05 GEMM family (``csrc/gemm/umma_gemm.cu``).

All tensors are bf16, 2-D, with a contiguous last dimension.  An operand is passed either
*K-major* (``[rows = M or N, cols = K]``) or *MN-major* (``[rows = K, cols = M or N]``); the
kernel builds the matching TMA boxes and shared-memory descriptors, so neither layout needs
a transpose copy.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _native as nv
from .tile_config import get_kernel_config


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with a contiguous last dim, got {tuple(t.shape)} "
                         f"strides {t.stride()}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bf16")
    if (t.stride(0) * 2) % 16 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"{name} must be 16-byte aligned with a 16-byte-multiple row pitch")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def fill_gemm_args(
    *,
    a: torch.Tensor,
    b: torch.Tensor,
    out: torch.Tensor,
    M: int,
    N: int,
    K: int,
    a_mn: bool = False,
    b_mn: bool = False,
    a2: Optional[torch.Tensor] = None,
    b2: Optional[torch.Tensor] = None,
    b2_mn: bool = False,
    K2: int = 0,
    bn: int = 256,
    nacc: int = 1,
    epi: int = nv.EPI_BF16,
    mask_a: bool = False,
    tile_adapter: Optional[torch.Tensor] = None,
    b_adapter_rows: int = 0,
    b2_adapter_rows: int = 0,
    seg_tiles: Optional[torch.Tensor] = None,
    ldo: Optional[int] = None,
    out_transposed: bool = False,
    out_adapter_stride: int = 0,
    adapter_scale: Optional[torch.Tensor] = None,
    scale: float = 1.0,
    bias: Optional[torch.Tensor] = None,
    adapter_thresh16: Optional[torch.Tensor] = None,
    adapter_inv_keep: Optional[torch.Tensor] = None,
    thresh16: int = 0,
    inv_keep: float = 1.0,
    seed: int = 0,
    stream_id: int = 0,
    row_offset: int = 0,
    col_offset: int = 0,
    group_m: Optional[int] = None,
    max_ctas: Optional[int] = None,
    tuned: Optional[str] = None,
) -> nv.LfGemmArgs:
    """Describe one GEMM launch (operands, epilogue, dropout, scheduling) as a
    :class:`LfGemmArgs` for the current stream.  ``tuned`` names the kernel family of the
    launch (``fwd`` / ``dx`` / ``dx_dropout``): scheduling parameters the caller leaves open are
    then taken from the tuned table (``ops/tile_config.py``) for this GPU and shape."""
    if tuned is not None and (group_m is None or max_ctas is None):
        cfg = get_kernel_config(tuned, M, K, N)
        group_m = cfg.group_m if group_m is None else group_m
        max_ctas = cfg.max_ctas if max_ctas is None else max_ctas
    group_m = 8 if group_m is None else group_m
    max_ctas = 0 if max_ctas is None else max_ctas
    _check2d(a, "a")
    args = nv.LfGemmArgs()
    args.a, args.a_rows, args.a_cols, args.a_ld = a.data_ptr(), a.shape[0], a.shape[1], a.stride(0)
    if hasattr(b, "packed"):
        # NF4 weight: the packed bytes stand in for the bf16 [rows, cols] matrix
        args.b, args.b_rows, args.b_cols, args.b_ld = b.packed.data_ptr(), b.shape[0], b.shape[1], b.shape[1]
    else:
        _check2d(b, "b")
        args.b, args.b_rows, args.b_cols, args.b_ld = b.data_ptr(), b.shape[0], b.shape[1], b.stride(0)
    if K2 > 0:
        _check2d(a2, "a2")
        _check2d(b2, "b2")
        args.a2, args.a2_rows, args.a2_cols, args.a2_ld = (
            a2.data_ptr(), a2.shape[0], a2.shape[1], a2.stride(0))
        args.b2, args.b2_rows, args.b2_cols, args.b2_ld = (
            b2.data_ptr(), b2.shape[0], b2.shape[1], b2.stride(0))
    args.tile_adapter = _ptr(tile_adapter)
    if seg_tiles is not None:
        if seg_tiles.dtype != torch.int32 or seg_tiles.dim() != 2 or seg_tiles.shape[1] != 4:
            raise ValueError("seg_tiles must be int32 [n, 4]")
        args.seg_tiles = seg_tiles.data_ptr()
        args.num_seg_tiles = seg_tiles.shape[0]
    args.out = out.data_ptr()
    args.ldo = out.stride(0) if ldo is None else ldo
    args.out_adapter_stride = out_adapter_stride
    args.adapter_scale = _ptr(adapter_scale)
    args.bias = _ptr(bias)
    args.adapter_thresh16 = _ptr(adapter_thresh16)
    args.adapter_inv_keep = _ptr(adapter_inv_keep)
    args.err = nv.err_word(a.device).data_ptr()
    args.stream = nv.current_stream_ptr()
    args.a_mn, args.b_mn, args.b2_mn = int(a_mn), int(b_mn), int(b2_mn)
    args.M, args.N, args.K, args.K2 = M, N, K, K2
    args.bn, args.nacc, args.epi, args.mask_a = bn, nacc, epi, int(mask_a)
    args.b_adapter_rows, args.b2_adapter_rows = b_adapter_rows, b2_adapter_rows
    args.out_transposed = int(out_transposed)
    args.scale = scale
    args.inv_keep = inv_keep
    args.thresh16 = thresh16
    args.seed_lo = seed & 0xFFFFFFFF
    args.seed_hi = (seed >> 32) & 0xFFFFFFFF
    args.stream_id = stream_id & 0xFFFFFFFF
    args.row_offset, args.col_offset = row_offset, col_offset
    args.group_m, args.max_ctas = group_m, max_ctas
    # keep the operand tensors alive until the struct has been consumed
    args._keepalive = (a, b, a2, b2, out, tile_adapter, seg_tiles, adapter_scale, bias,
                       adapter_thresh16, adapter_inv_keep)
    return args


# CTA-pair (tcgen05 cta_group::2, 256 x 256 tiles) kernels for the big GEMMs; "0" disables.
_PAIR = os.environ.get("LORAFUSION_B200_PAIR", "1") == "1"
_PAIR_MIN_ROWS = 512


def set_pair_kernels(enabled: bool) -> None:
    """Route eligible GEMMs (256-wide tiles, dense mode, no in-smem dropout) to the CTA-pair
    kernels of ``csrc/gemm/umma_gemm_pair.cu`` (True) or keep everything on the single-CTA
    template (False)."""
    global _PAIR
    _PAIR = bool(enabled)


def launch_gemm(pair: Optional[bool] = None, **kwargs) -> None:
    """Fill :class:`LfGemmArgs` (see :func:`fill_gemm_args`) and launch on the current stream.
    ``pair`` overrides the module default for trying the CTA-pair kernel first.  When ``b`` is
    an :class:`~lorafusion_b200.ops.nf4.NF4Weight` the kernel that expands NF4 inside its main
    loop runs (``lf_gemm_nf4``)."""
    lib = nv.cuda_lib()
    args = fill_gemm_args(**kwargs)
    nv.note_launch()
    qw = kwargs["b"]
    if hasattr(qw, "packed"):
        q = nv.LfNf4Args()
        scales = qw.fp32_block_scales()
        q.block_scales, q.w_rows, q.w_cols = scales.data_ptr(), qw.shape[0], qw.shape[1]
        rc = lib.lf_gemm_nf4(C.byref(args), C.byref(q))
        if rc != 0:
            raise RuntimeError(f"lf_gemm_nf4 failed with code {rc}")
        return
    use_pair = _PAIR if pair is None else pair
    if use_pair and args.bn == 256 and args.M >= _PAIR_MIN_ROWS and not args.a_mn and not args.mask_a \
            and not args.seg_tiles:
        rc = lib.lf_gemm_pair(C.byref(args))
        if rc == 0:
            return
        if rc != -5:
            raise RuntimeError(f"lf_gemm_pair failed with code {rc}")
    rc = lib.lf_gemm(C.byref(args))
    if rc != 0:
        raise RuntimeError(f"lf_gemm failed with code {rc}")


def _pick_bn(n: int) -> int:
    return 256 if n >= 256 else 128


def gemm_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[M, K] @ b[N, K]^T (+ bias[N])`` -> bf16 ``[M, N]``."""
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    launch_gemm(a=a, b=b, out=out, M=M, N=N, K=K, bn=_pick_bn(N), bias=bias)
    return out


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a[M, K] @ b[K, N]`` -> bf16 ``[M, N]`` (``b`` consumed MN-major, no transpose copy)."""
    M, K = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    launch_gemm(a=a, b=b, out=out, M=M, N=N, K=K, b_mn=True, b2_mn=True, bn=_pick_bn(N))
    return out
