"""ZeRO-3 / FSDP-style baseline: the frozen base weights are sharded over the data-parallel
group and every layer is all-gathered right before its forward and again before its backward.

This is the reference's "Megatron-LM-FSDP" arm (``--use_fsdp``: Megatron's
``TorchFullyShardedDataParallel`` around every decoder layer,
``benchmarks_paper/bench_multi_gpu.py:131-134``, ``lorafusion/utils/module.py:28``), rebuilt
inside this runtime so that it can be measured on the same GPUs as the product path.  It is a
BASELINE: the collective is a plain NCCL all-gather (no fusion with the GEMMs), prefetched one
layer ahead so that it overlaps the previous layer's compute, which is what FSDP does.

Memory: a rank holds ``1 / dp`` of every layer's weights plus two gather buffers of one full
layer; LoRA adapters, their gradients and optimizer state are handled exactly as under plain
data parallelism (they are tiny next to the base).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..ops.nf4 import NF4Weight
from .config import AdapterSpec, ModelConfig
from .decoder import DecoderStage, LayerWeights

_ALIGN = 256  # every tensor starts on a 256-byte boundary inside the flat layer buffer (TMA needs 16)


@dataclass
class _Piece:
    """One tensor of a layer inside the layer's flat byte buffer."""

    proj: str          # qkv | o | gate_up | down
    field: str         # "dense" (bf16 weight) | "packed" | "absmax" | "absmax_q"
    offset: int
    nbytes: int
    shape: tuple
    dtype: torch.dtype


@dataclass
class _ShardedLayer:
    shard: torch.Tensor            # uint8 [per_rank]
    pieces: list
    small: dict                    # proj -> NF4 side tensors that stay replicated (code table, nested scales, ...)
    total: int                     # bytes of the flat layer buffer (padded to world x per_rank)
    ln1: torch.Tensor
    ln2: torch.Tensor
    qkv_bias: Optional[torch.Tensor]


class FsdpDecoderStage(DecoderStage):
    """A :class:`DecoderStage` whose frozen weights live sharded over ``shard_group``."""

    def __init__(self, cfg: ModelConfig, adapters: Sequence[AdapterSpec], device, shard_group, **kw):
        self.shard_group = shard_group
        self.shard_world = dist.get_world_size(shard_group) if shard_group is not None else 1
        self.shard_rank = dist.get_rank(shard_group) if shard_group is not None else 0
        self._sharded: list = []
        self._buffers: list = []
        self._inflight: dict = {}   # layer -> (buffer index, work handle)
        self._next_buf = 0
        self.gathered_bytes = 0
        super().__init__(cfg, adapters, device, **kw)
        biggest = max((s.total for s in self._sharded), default=0)
        self._buffers = [torch.empty(biggest, dtype=torch.uint8, device=self.device) for _ in range(2)]

    # ------------------------------------------------------------------ sharding at construction
    def _adopt_layer(self, li: int, lw: LayerWeights) -> LayerWeights:
        pieces, small, chunks, off = [], {}, [], 0

        def add(proj, field, t):
            nonlocal off
            raw = t.contiguous().view(torch.uint8).reshape(-1)
            pieces.append(_Piece(proj, field, off, raw.numel(), tuple(t.shape), t.dtype))
            pad = (-raw.numel()) % _ALIGN
            chunks.append(raw)
            if pad:
                chunks.append(torch.zeros(pad, dtype=torch.uint8, device=raw.device))
            off += raw.numel() + pad

        for proj in ("qkv", "o", "gate_up", "down"):
            w = getattr(lw, proj)
            if isinstance(w, NF4Weight):
                add(proj, "packed", w.packed)
                if w.absmax is not None:
                    add(proj, "absmax", w.absmax)
                if w.absmax_q is not None:
                    add(proj, "absmax_q", w.absmax_q)
                small[proj] = dict(shape=w.shape, code256=w.code256, nested=w.nested, offset=w.offset)
            else:
                add(proj, "dense", w)
        world = self.shard_world
        per = ((off + world - 1) // world + _ALIGN - 1) // _ALIGN * _ALIGN
        flat = torch.cat(chunks)
        if flat.numel() < per * world:
            flat = torch.cat([flat, torch.zeros(per * world - flat.numel(), dtype=torch.uint8, device=flat.device)])
        shard = flat[self.shard_rank * per:(self.shard_rank + 1) * per].clone()
        self._sharded.append(_ShardedLayer(shard, pieces, small, per * world, lw.ln1, lw.ln2, lw.qkv_bias))
        del flat, chunks
        # the full weights of this layer are released when the caller drops `lw`
        return LayerWeights(ln1=lw.ln1, ln2=lw.ln2, qkv=None, o=None, gate_up=None, down=None, qkv_bias=lw.qkv_bias)

    def base_weight_bytes(self) -> int:
        """Bytes of frozen weights THIS rank stores."""
        return sum(s.shard.numel() for s in self._sharded)

    # ------------------------------------------------------------------ gathering
    def _start_gather(self, li: int) -> None:
        if li in self._inflight or not (0 <= li < len(self._sharded)):
            return
        sl = self._sharded[li]
        idx = self._next_buf
        self._next_buf = (idx + 1) % len(self._buffers)
        for other, (b, _) in list(self._inflight.items()):
            if b == idx:  # the buffer is being reused: its earlier content is no longer wanted
                del self._inflight[other]
        out = self._buffers[idx][:sl.total]
        work = None
        if self.shard_world > 1:
            # async: NCCL's stream first waits for what is queued on the compute stream so far
            # (the last user of this buffer), then runs next to the compute queued after this call
            work = dist.all_gather_into_tensor(out, sl.shard, group=self.shard_group, async_op=True)
        else:
            out.copy_(sl.shard)
        self.gathered_bytes += sl.total
        self._inflight[li] = (idx, work)

    def _materialise(self, li: int) -> LayerWeights:
        self._start_gather(li)
        idx, work = self._inflight.pop(li)
        if work is not None:
            work.wait()   # the compute stream waits for the gather; the host does not block
        sl, buf = self._sharded[li], self._buffers[idx]
        got: dict = {}
        for p in sl.pieces:
            got.setdefault(p.proj, {})[p.field] = buf[p.offset:p.offset + p.nbytes].view(p.dtype).view(p.shape)
        weights = {}
        for proj, fields in got.items():
            if "dense" in fields:
                weights[proj] = fields["dense"]
            else:
                sm = sl.small[proj]
                weights[proj] = NF4Weight(fields["packed"], sm["shape"], fields.get("absmax"), fields.get("absmax_q"),
                                          sm["code256"], sm["nested"], sm["offset"])
        return LayerWeights(ln1=sl.ln1, ln2=sl.ln2, qkv_bias=sl.qkv_bias, **weights)

    # ------------------------------------------------------------------ layer hooks
    def _layer_forward(self, li, res, delta, batch, keep):
        if self.layers[li].qkv is not None:   # called from this layer's backward (recomputation)
            return super()._layer_forward(li, res, delta, batch, keep)
        self.layers[li] = self._materialise(li)
        self._start_gather(li + 1)                      # prefetch: overlaps this layer's compute
        try:
            return super()._layer_forward(li, res, delta, batch, keep)
        finally:
            sl = self._sharded[li]
            self.layers[li] = LayerWeights(ln1=sl.ln1, ln2=sl.ln2, qkv=None, o=None, gate_up=None, down=None,
                                           qkv_bias=sl.qkv_bias)

    def _layer_backward(self, li, saved, dh, batch, need_input_grad=True):
        self.layers[li] = self._materialise(li)
        self._start_gather(li - 1)
        try:
            return super()._layer_backward(li, saved, dh, batch, need_input_grad=need_input_grad)
        finally:
            sl = self._sharded[li]
            self.layers[li] = LayerWeights(ln1=sl.ln1, ln2=sl.ln2, qkv=None, o=None, gate_up=None, down=None,
                                           qkv_bias=sl.qkv_bias)
