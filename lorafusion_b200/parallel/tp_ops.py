"""Tensor-parallel fused ops: all-gather -> fused base+LoRA GEMM and fused base+LoRA GEMM ->
reduce-scatter, each as ONE kernel that moves data over NVLink peer memory while it computes
(``csrc/gemm/umma_gemm.cu``, ``TP`` template parameter).

The reference has no tensor parallelism (``tp`` is hard-wired to 1,
``benchmarks_paper/bench_multi_gpu.py:624``); these ops exist for the TP x PP configurations
of the 32B / 70B models.  Activations between them are sequence-parallel: every TP rank holds
``T / tp`` token rows of the residual stream.

``TpContext`` owns the symmetric buffers (allocated once, reused by every layer):

* ``gather`` ``[T, K_max]``  -- destination of the all-gathered A operand (a rank writes its
  own shard in place, peers push theirs during the consuming kernel), ``gather2`` for the
  LoRA ``S'`` / ``dS`` operand, ``ag_flags`` one flag per (source rank, row tile);
* ``rs_stage`` ``[T, N_max]`` -- where this rank keeps its partial output tiles of ALL rows; the
  owner of a row pulls it from every rank's stage.  ``rs_cnt`` one epoch flag per (source rank,
  row tile, column tile), raised in the owner's memory when the partial tile is complete.

Flags carry a per-context epoch that grows with every call, so microbatches of different
sizes can reuse the same flag words.

Buffer reuse is safe without extra barriers because all-gather and reduce-scatter uses
alternate: a rank can only reach the next all-gather after receiving every peer's partials of
the reduce-scatter in between, which those peers send after they finished reading the
previous gather (and vice versa).
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _native as nv
from ..ops.gemm import fill_gemm_args
from .symmetric import SymmetricBuffer, allocate_symmetric, local_buffer

TILE = 128
# CTA-pair variants of the fused kernels; "0" keeps everything on the single-CTA template
_PAIR_TP = os.environ.get("LORAFUSION_B200_PAIR_TP", "1") == "1"


def set_pair_tp_kernels(enabled: bool) -> None:
    """Route the tensor-parallel fused GEMMs to the CTA-pair kernels (True) or to the single-CTA
    template (False); shapes the pair kernels do not cover always use the template."""
    global _PAIR_TP
    _PAIR_TP = bool(enabled)


class LfTpArgs(C.Structure):
    _fields_ = [
        ("ag_flags", C.c_void_p),
        ("ag_peer_flags", C.c_void_p * 8),
        ("ag_src", C.c_void_p),
        ("ag_ld", C.c_int64),
        ("ag_peer_dst", C.c_void_p * 8),
        ("ag2_src", C.c_void_p),
        ("ag2_ld", C.c_int64),
        ("ag2_peer_dst", C.c_void_p * 8),
        ("rs_peer_stage", C.c_void_p * 8),
        ("rs_peer_cnt", C.c_void_p * 8),
        ("rs_cnt", C.c_void_p),
        ("rs_out", C.c_void_p),
        ("rs_ldo", C.c_int64),
        ("rs_residual", C.c_void_p),
        ("mode", C.c_int32), ("rank", C.c_int32), ("world", C.c_int32), ("tiles_per_shard", C.c_int32),
        ("epoch", C.c_int32), ("rs_target", C.c_int32), ("ag_cols", C.c_int32), ("ag2_cols", C.c_int32),
    ]


class TpContext:
    def __init__(self, group, device, *, max_tokens: int, max_features: int, max_rank_width: int = 256):
        self.group = group
        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        if max_tokens % (TILE * self.world):
            raise ValueError("token count must be a multiple of 128 * tp")
        self.max_tokens, self.max_features, self.max_rank_width = max_tokens, max_features, max_rank_width
        alloc = (lambda n, dt: allocate_symmetric(n, dt, self.device, group)) if self.world > 1 else \
            (lambda n, dt: local_buffer(n, dt, self.device))
        self.gather: SymmetricBuffer = alloc(max_tokens * max_features, torch.bfloat16)
        self.gather2: SymmetricBuffer = alloc(max_tokens * max_rank_width, torch.bfloat16)
        self.rs_stage: SymmetricBuffer = alloc(max_tokens * max_features, torch.bfloat16)
        n_flags = self.world * (max_tokens // TILE)
        # flags [n_flags] followed by this rank's slice-arrival counters [max_tokens / 128]
        self.n_flags = n_flags
        self.ag_flags: SymmetricBuffer = alloc(n_flags + max_tokens // TILE, torch.int32)
        # one flag per (source rank, row tile, 256-column tile) of a reduce-scatter
        self.rs_cnt: SymmetricBuffer = alloc(n_flags * ((max_features + 255) // 256), torch.int32)
        self.ag_flags.tensor.zero_()
        self.rs_cnt.tensor.zero_()
        self.epoch = 0
        self.rs_total = 0
        self._last_mode = 0
        self._fence_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group)

    # ---- one-GPU loop-back: run the copy / reduce warps without a second GPU ----------------
    @classmethod
    def loopback(cls, device, *, world: int = 2, max_tokens: int, max_features: int,
                 max_rank_width: int = 256) -> "TpContext":
        """A context that makes ONE GPU act as rank 0 of ``world`` ranks: every peer pointer
        leads back to this GPU's own memory.  The kernels then run their communication warps for
        real -- shard pushes, flag raises, flag waits, peer pulls -- over local addresses, which
        is how they are tested and profiled where only one GPU is at hand.  The part of the
        other ranks is played by the host BEFORE each launch (:meth:`loopback_arm_gather`,
        :meth:`loopback_arm_reduce`): it puts their data in place and raises their flags, so the
        kernel never waits for anything that is not already there."""
        self = cls(None, device, max_tokens=max_tokens * 1, max_features=max_features, max_rank_width=max_rank_width)
        if max_tokens % (TILE * world):
            raise ValueError("token count must be a multiple of 128 * world")
        self.world, self.rank, self.is_loopback = world, 0, True
        dev = self.device
        n_flags = world * (max_tokens // TILE)
        self.n_flags = n_flags
        self.ag_flags = local_buffer(n_flags + max_tokens // TILE, torch.int32, dev)
        self.rs_cnt = local_buffer(n_flags * ((max_features + 255) // 256), torch.int32, dev)
        # pushes of the own shard land on the own rows again; flags raised "at the peers" land in
        # the own flag array, in this rank's slots
        self.gather.peer_ptrs = [self.gather.tensor.data_ptr()] * world
        self.gather2.peer_ptrs = [self.gather2.tensor.data_ptr()] * world
        self.ag_flags.peer_ptrs = [self.ag_flags.tensor.data_ptr()] * world
        # partial tiles of the other ranks come from stand-in stages the host fills; completion
        # flags for rows owned by other ranks go to a scratch array nobody reads
        self.peer_stages = [self.rs_stage.tensor] + [torch.zeros_like(self.rs_stage.tensor) for _ in range(world - 1)]
        self.rs_stage.peer_ptrs = [t.data_ptr() for t in self.peer_stages]
        self._rs_scratch = torch.zeros_like(self.rs_cnt.tensor)
        self.rs_cnt.peer_ptrs = [self.rs_cnt.tensor.data_ptr()] + [self._rs_scratch.data_ptr()] * (world - 1)
        return self

    def loopback_arm_gather(self, tokens: int) -> None:
        """Before an ``ag_gemm`` in loop-back mode: the rows of the other ranks are already in the
        gather buffers (the caller wrote them); raise their flags for the coming call."""
        tps = tokens // self.world // TILE
        self.ag_flags.tensor[tps:self.world * tps] = self.epoch + 1

    def loopback_arm_reduce(self, tokens: int, n: int, partials: list) -> None:
        """Before a ``gemm_rs`` in loop-back mode: ``partials[r - 1]`` = the ``[tokens, n]`` partial
        product rank ``r`` would have left in its stage; raise those ranks' completion flags for
        the rows this rank owns."""
        tps = tokens // self.world // TILE
        nnt = (n + 255) // 256
        for r, part in enumerate(partials, start=1):
            self.peer_stages[r][:tokens * n].view(tokens, n).copy_(part)
        self.rs_cnt.tensor[tps * nnt:self.world * tps * nnt] = self.epoch + 1

    def order(self, mode: int) -> None:
        """The reuse argument for the gather / stage buffers needs all-gather and
        reduce-scatter uses to alternate.  When the same kind is requested twice in a row
        (e.g. the last backward op of one microbatch and the first forward op of the next are
        both all-gathers) a one-word all-reduce orders the ranks in between."""
        if self.world > 1 and mode == self._last_mode and not getattr(self, "is_loopback", False):
            dist.all_reduce(self._fence_word, group=self.group)
        self._last_mode = mode

    # ---- views a producer kernel writes its own shard into ---------------------------------
    def shard_rows(self, tokens: int) -> tuple:
        ms = tokens // self.world
        return self.rank * ms, (self.rank + 1) * ms

    def gather_view(self, tokens: int, cols: int) -> torch.Tensor:
        return self.gather.tensor[:tokens * cols].view(tokens, cols)

    def gather2_view(self, tokens: int, cols: int) -> torch.Tensor:
        return self.gather2.tensor[:tokens * cols].view(tokens, cols)

    def own_gather_rows(self, tokens: int, cols: int) -> torch.Tensor:
        r0, r1 = self.shard_rows(tokens)
        return self.gather_view(tokens, cols)[r0:r1]

    def own_gather2_rows(self, tokens: int, cols: int) -> torch.Tensor:
        r0, r1 = self.shard_rows(tokens)
        return self.gather2_view(tokens, cols)[r0:r1]

    def _base_args(self, tokens: int) -> LfTpArgs:
        t = LfTpArgs()
        t.rank, t.world = self.rank, self.world
        t.tiles_per_shard = tokens // self.world // TILE
        return t


def _launch(gemm_kwargs: dict, tp: LfTpArgs) -> None:
    lib = nv.cuda_lib()
    if not getattr(lib, "_lf_tp_declared", False):
        lib.lf_gemm_tp.argtypes = [C.POINTER(nv.LfGemmArgs), C.POINTER(LfTpArgs)]
        lib.lf_gemm_tp.restype = C.c_int
        lib._lf_tp_declared = True
    args = fill_gemm_args(**gemm_kwargs)
    nv.note_launch()
    qw = gemm_kwargs["b"]
    if hasattr(qw, "packed"):  # NF4 weight shard, expanded inside the kernel's main loop
        if not getattr(lib, "_lf_tp_nf4_declared", False):
            lib.lf_gemm_tp_nf4.argtypes = [C.POINTER(nv.LfGemmArgs), C.POINTER(LfTpArgs), C.POINTER(nv.LfNf4Args)]
            lib.lf_gemm_tp_nf4.restype = C.c_int
            lib._lf_tp_nf4_declared = True
        q = nv.LfNf4Args()
        scales = qw.fp32_block_scales()
        q.block_scales, q.w_rows, q.w_cols = scales.data_ptr(), qw.shape[0], qw.shape[1]
        rc = lib.lf_gemm_tp_nf4(C.byref(args), C.byref(tp), C.byref(q))
        if rc != 0:
            raise RuntimeError(f"lf_gemm_tp_nf4 failed with code {rc}")
        return
    if _PAIR_TP:
        # CTA-pair (256 x 256 tile, tcgen05 cta_group::2) variant first; -5 = shape not covered
        if not getattr(lib, "_lf_pair_tp_declared", False):
            lib.lf_gemm_pair_tp.argtypes = [C.POINTER(nv.LfGemmArgs), C.POINTER(LfTpArgs)]
            lib.lf_gemm_pair_tp.restype = C.c_int
            lib._lf_pair_tp_declared = True
        rc = lib.lf_gemm_pair_tp(C.byref(args), C.byref(tp))
        if rc == 0:
            return
        if rc != -5:
            raise RuntimeError(f"lf_gemm_pair_tp failed with code {rc}")
    rc = lib.lf_gemm_tp(C.byref(args), C.byref(tp))
    if rc != 0:
        raise RuntimeError(f"lf_gemm_tp failed with code {rc}")


def ag_gemm(ctx: TpContext, tokens: int, k: int, w: torch.Tensor, *, w_mn: bool = False,
            slab_cols: int = 0, b2: Optional[torch.Tensor] = None, b2_adapter_rows: int = 0,
            tile_adapter: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
            dropout_kwargs: Optional[dict] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[T, N] = gathered_A[T, k] @ W (+ gathered_slab[T, R] @ B2)``.

    The caller has already written this rank's rows of A into ``ctx.own_gather_rows(tokens,
    k)`` (and of the slab operand into ``ctx.own_gather2_rows(tokens, slab_cols)``); the
    kernel pushes them to the peers and consumes the peers' rows as they land.  ``w`` is
    ``[N, k]`` (``w_mn=False``) or ``[k, N]`` consumed MN-major (``w_mn=True``, used for
    ``dY_full @ W_shard`` in the backward); an :class:`~lorafusion_b200.ops.nf4.NF4Weight` is
    expanded inside the kernel's main loop."""
    a = ctx.gather_view(tokens, k)
    N = w.shape[1] if w_mn else w.shape[0]
    if out is None:
        out = torch.empty((tokens, N), dtype=torch.bfloat16, device=ctx.device)
    ctx.epoch += 1
    ctx.order(1)
    tp = ctx._base_args(tokens)
    tp.mode, tp.epoch = 1, ctx.epoch
    tp.ag_flags = ctx.ag_flags.tensor.data_ptr()
    tp.rs_target = ctx.n_flags  # offset (ints) of the arrival counters behind the flags
    tp.ag_src, tp.ag_ld, tp.ag_cols = a.data_ptr(), k, k
    for r in range(ctx.world):
        tp.ag_peer_flags[r] = ctx.ag_flags.peer_ptrs[r]
        tp.ag_peer_dst[r] = ctx.gather.peer_ptrs[r]
        tp.ag2_peer_dst[r] = ctx.gather2.peer_ptrs[r]
    kw = dict(a=a, b=w, out=out, M=tokens, N=N, K=k, b_mn=w_mn, b2_mn=w_mn, bn=256, bias=bias,
              tile_adapter=tile_adapter)
    if slab_cols:
        a2 = ctx.gather2_view(tokens, slab_cols)
        tp.ag2_src, tp.ag2_ld, tp.ag2_cols = a2.data_ptr(), slab_cols, slab_cols
        kw.update(a2=a2, b2=b2.reshape(-1, b2.shape[-1]), K2=slab_cols, b2_adapter_rows=b2_adapter_rows)
    if dropout_kwargs:
        kw.update(nacc=2, epi=nv.EPI_BF16_DROPMIX, **dropout_kwargs)
    _launch(kw, tp)
    return out


def gemm_rs(ctx: TpContext, x: torch.Tensor, w: torch.Tensor, *, w_mn: bool = False,
            s: Optional[torch.Tensor] = None, b2: Optional[torch.Tensor] = None, b2_adapter_rows: int = 0,
            tile_adapter: Optional[torch.Tensor] = None, dropout_kwargs: Optional[dict] = None,
            residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[T / tp, N] = reduce_scatter_over_tp(x[T, k_local] @ W_local (+ s @ B2))
    (+ residual)``: this rank's rows of the sum of all ranks' partial products."""
    tokens, k = x.shape
    N = w.shape[1] if w_mn else w.shape[0]
    ms = tokens // ctx.world
    if out is None:
        out = torch.empty((ms, N), dtype=torch.bfloat16, device=ctx.device)
    if N > ctx.max_features or tokens > ctx.max_tokens:
        raise ValueError("reduce-scatter larger than the TP context was sized for")
    ctx.epoch += 1
    ctx.order(2)
    tp = ctx._base_args(tokens)
    tp.mode, tp.epoch = 2, ctx.epoch
    tp.rs_cnt = ctx.rs_cnt.tensor.data_ptr()
    tp.rs_out, tp.rs_ldo = out.data_ptr(), out.stride(0)
    tp.rs_residual = residual.data_ptr() if residual is not None else None
    for r in range(ctx.world):
        tp.rs_peer_stage[r] = ctx.rs_stage.peer_ptrs[r]
        tp.rs_peer_cnt[r] = ctx.rs_cnt.peer_ptrs[r]
    # `out` of the GEMM args is unused in this mode but must be a valid pointer
    kw = dict(a=x, b=w, out=out, M=tokens, N=N, K=k, b_mn=w_mn, b2_mn=w_mn, bn=256, tile_adapter=tile_adapter,
              ldo=N)
    if s is not None:
        kw.update(a2=s, b2=b2.reshape(-1, b2.shape[-1]), K2=s.shape[1], b2_adapter_rows=b2_adapter_rows)
    if dropout_kwargs:
        kw.update(nacc=2, epi=nv.EPI_BF16_DROPMIX, **dropout_kwargs)
    _launch(kw, tp)
    return out
