"""Own decoder-only transformer (Llama / Qwen2 shaped) with a hand-written training engine.

The reference monkey-patches HF models + PEFT and lets autograd drive the backward
(``lorafusion/train/training_utils.py:533-629``, ``lorafusion/patch/*``).  Here the model
is a set of frozen weights (bf16 or NF4) plus a :class:`LoRAArena`, and forward / backward
are written out explicitly over the sm_100a kernels:

    rmsnorm(+residual) -> fused LoRA linear (q|k|v merged) -> RoPE in place -> causal varlen
    attention -> fused LoRA linear (o) -> rmsnorm(+residual) -> fused LoRA linear (gate|up
    merged) -> SwiGLU -> fused LoRA linear (down)

Because the base is frozen there are no weight gradients outside the adapters, and because
the dropout mask is counter-based a layer can be recomputed in the backward from nothing but
its input (activation recomputation, the counterpart of the reference's selective gradient
checkpointing, ``training_utils.py:632-732``).  A model instance owns a contiguous range of
layers (a pipeline stage); the first stage owns the embedding, the last the final norm and
the lm_head, whose loss is computed chunk by chunk together with its backward so that the
[tokens, vocab] logits never exist in full.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..ops import elementwise as ew
from ..ops import attention as att
from ..ops.batch_info import MultiLoRABatchInfo
from ..ops.gemm import gemm_nn, gemm_nt
from ..ops.lora import lora_linear_backward, lora_linear_forward
from ..ops.nf4 import NF4Weight, quantize_nf4
from .adapters import LoRAArena
from .config import AdapterSpec, ModelConfig

PROJ_STREAM = {"qkv": 0, "o": 1, "gate_up": 2, "down": 3}


@dataclass
class PackedBatch:
    """One packed microbatch on the device.

    ``input_ids`` / ``labels`` / ``position_ids`` are int32 ``[T]`` (labels already shifted,
    ``-100`` = ignored); ``cu_seqlens`` holds host ints; ``info`` maps 128-token tiles to
    adapters.  ``T`` is a multiple of 128 because every adapter segment is padded to one."""

    input_ids: torch.Tensor
    labels: torch.Tensor
    position_ids: torch.Tensor
    cu_seqlens: list
    attn_tiles: att.AttnTiles
    info: MultiLoRABatchInfo
    num_real_tokens: int = 0
    num_loss_tokens: int = 0

    @property
    def num_tokens(self) -> int:
        return int(self.input_ids.shape[0])


def rope_tables(cfg: ModelConfig, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin ``[max_position, head_dim / 2]`` in fp32, with Llama-3.1 scaling if set."""
    d = cfg.head_dim
    inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    sc = cfg.rope_scaling
    if sc is not None:
        low_wl = sc.original_max_position / sc.low_freq_factor
        high_wl = sc.original_max_position / sc.high_freq_factor
        wl = 2 * math.pi / inv_freq
        smooth = (sc.original_max_position / wl - sc.low_freq_factor) / (sc.high_freq_factor - sc.low_freq_factor)
        scaled = torch.where(wl > low_wl, inv_freq / sc.factor, inv_freq)
        mid = (wl <= low_wl) & (wl >= high_wl)
        scaled = torch.where(mid, (1 - smooth) * inv_freq / sc.factor + smooth * inv_freq, scaled)
        inv_freq = scaled
    ang = torch.arange(cfg.max_position, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    qkv: object  # bf16 tensor or NF4Weight
    o: object
    gate_up: object
    down: object
    qkv_bias: Optional[torch.Tensor] = None


@dataclass
class LayerSaved:
    """What a layer keeps for its backward.  With recomputation only ``h_in`` is kept
    between forward and backward; the rest is rebuilt right before it is needed."""

    h_in: torch.Tensor
    full: Optional[dict] = None


class DecoderStage:
    """Layers ``[layer_start, layer_end)`` of a decoder, on one GPU."""

    def __init__(self, cfg: ModelConfig, adapters: Sequence[AdapterSpec], device, *,
                 layer_start: int = 0, layer_end: Optional[int] = None, quantize: bool = False,
                 double_quant: bool = True, init_std: float = 0.02, init_b_std: float = 0.0,
                 seed: int = 0, recompute=True, with_optimizer_state: bool = True,
                 head_chunk_tokens: int = 2048, max_inflight: int = 1, reserve_bytes: int = 12 << 30,
                 shared_alloc=None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.layer_start = layer_start
        self.layer_end = cfg.num_layers if layer_end is None else layer_end
        self.is_first = self.layer_start == 0
        self.is_last = self.layer_end == cfg.num_layers
        self.quantize = quantize
        self.recompute = recompute  # True | False | "auto"
        self.max_inflight = max(1, max_inflight)
        self.reserve_bytes = reserve_bytes
        self._keep_plan: dict = {}
        self._modes_plan: Optional[list] = None
        self._modes_tokens = 0
        self.force_keep_modes: Optional[list] = None  # tests / experiments: per-layer keep mode
        self.offload_enabled = False      # park gate|up outputs in pinned host memory
        self.offload_host_budget: Optional[int] = None  # bytes; None = share of MemAvailable
        self.offload_max_layers: Optional[int] = None   # what the PCIe link drains during one forward
        self._offloader = None
        self.head_chunk_tokens = head_chunk_tokens
        self.training = True
        self.adapters = list(adapters)
        g = torch.Generator(device=self.device).manual_seed(seed + 1000 * layer_start)
        h, i = cfg.hidden_size, cfg.intermediate_size

        def rnd(*shape, std=init_std):
            return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * std).to(torch.bfloat16)

        def frozen(n, k):
            w = rnd(n, k)
            if quantize:
                q = quantize_nf4(w, double_quant=double_quant)
                del w
                return q
            return w

        self.layers: list[LayerWeights] = []
        for _ in range(self.layer_start, self.layer_end):
            self.layers.append(self._adopt_layer(len(self.layers), LayerWeights(
                ln1=torch.ones(h, dtype=torch.bfloat16, device=self.device),
                ln2=torch.ones(h, dtype=torch.bfloat16, device=self.device),
                qkv=frozen(cfg.qkv_size, h), o=frozen(h, cfg.q_size),
                gate_up=frozen(2 * i, h), down=frozen(h, i),
                qkv_bias=rnd(cfg.qkv_size) if cfg.qkv_bias else None)))
        self.embed = rnd(cfg.vocab_size, h) if self.is_first else None
        self.final_norm = torch.ones(h, dtype=torch.bfloat16, device=self.device) if self.is_last else None
        self.lm_head = rnd(cfg.vocab_size, h) if self.is_last else None
        self.cos, self.sin = rope_tables(cfg, self.device)
        self.arena = LoRAArena(cfg, self.adapters, range(self.layer_start, self.layer_end), self.device,
                               init_b_std=init_b_std, seed=seed,
                               with_optimizer_state=with_optimizer_state,
                               shared_alloc=shared_alloc) if self.adapters else None

    def _adopt_layer(self, li: int, lw: LayerWeights) -> LayerWeights:
        """Hook called with every freshly initialised layer; a subclass may replace the
        weights by its own representation (e.g. a shard) before the next layer is created."""
        return lw

    def adopt_weights(self, full: "DecoderStage") -> "DecoderStage":
        """Make this stage a slice of ``full`` (a stage covering at least the same layers):
        frozen weights are shared, adapter weights are copied.  Used to compare a partitioned
        model with the unpartitioned one."""
        off = self.layer_start - full.layer_start
        if off < 0 or self.layer_end > full.layer_end:
            raise ValueError("the source stage does not cover these layers")
        self.layers = full.layers[off:off + (self.layer_end - self.layer_start)]
        if self.is_first:
            self.embed = full.embed
        if self.is_last:
            self.final_norm, self.lm_head = full.final_norm, full.lm_head
        if self.arena is not None:
            for i in range(len(self.adapters)):
                self.arena.import_adapter(i, full.arena.export_adapter(i))
        return self

    # ------------------------------------------------------------------ helpers
    def _stack(self, layer: int, proj: str):
        return self.arena.stack(layer, proj) if self.arena is not None else None

    @staticmethod
    def _sid(layer: int, proj: str) -> int:
        return layer * 8 + PROJ_STREAM[proj]

    def train(self, mode: bool = True):
        self.training = mode
        return self

    def base_weight_bytes(self) -> int:
        tot = 0
        for lw in self.layers:
            for w in (lw.qkv, lw.o, lw.gate_up, lw.down):
                tot += w.nbytes() if isinstance(w, NF4Weight) else w.numel() * w.element_size()
        return tot

    # ------------------------------------------------------------------ one layer
    def _layer_forward(self, li: int, res: Optional[torch.Tensor], delta: torch.Tensor,
                       batch: PackedBatch, keep: bool):
        """``(res, delta)`` -> ``(h_mid, d)`` with ``h_in = res + delta`` and the layer output
        ``h_mid + d``.  ``keep`` = store everything the backward needs."""
        cfg, lw, l = self.cfg, self.layers[li], self.layer_start + li
        info, tr = batch.info, self.training
        x1, h_in, rstd1 = ew.rmsnorm_fwd(delta, lw.ln1, cfg.rms_eps, res=res)
        qkv, s_qkv = lora_linear_forward(x1, lw.qkv, self._stack(l, "qkv"), info,
                                         stream_id=self._sid(l, "qkv"), bias=lw.qkv_bias, training=tr)
        ew.rope_inplace(qkv, batch.position_ids, self.cos, self.sin, cfg.num_heads + cfg.num_kv_heads,
                        cfg.head_dim)
        attn, lse = att.attention_forward(qkv, batch.attn_tiles, cfg.num_heads, cfg.num_kv_heads)
        o, s_o = lora_linear_forward(attn, lw.o, self._stack(l, "o"), info, stream_id=self._sid(l, "o"),
                                     training=tr)
        x2, h_mid, rstd2 = ew.rmsnorm_fwd(o, lw.ln2, cfg.rms_eps, res=h_in)
        gu, s_gu = lora_linear_forward(x2, lw.gate_up, self._stack(l, "gate_up"), info,
                                       stream_id=self._sid(l, "gate_up"), training=tr)
        act = ew.swiglu_fwd(gu)
        d, s_d = lora_linear_forward(act, lw.down, self._stack(l, "down"), info,
                                     stream_id=self._sid(l, "down"), training=tr)
        full = None
        if keep:
            full = dict(rstd1=rstd1, qkv=qkv, attn=attn, lse=lse, s_qkv=s_qkv, s_o=s_o,
                        h_mid=h_mid, rstd2=rstd2, s_gu=s_gu, s_d=s_d)
            if keep == "offload":  # gate|up goes to pinned host memory, overlapped with compute
                full["gu_off"] = self._get_offloader(gu.shape[0]).store(li, gu)
            elif keep != "nogu":  # "nogu" drops the (largest) gate|up projection output
                full["gu"] = gu
            if keep is True:  # "cheap" / "nogu" drop what one elementwise kernel can rebuild
                full.update(x1=x1, x2=x2, act=act)
        return h_mid, d, LayerSaved(h_in, full)

    def _layer_backward(self, li: int, saved: LayerSaved, dh: torch.Tensor, batch: PackedBatch,
                        need_input_grad: bool = True) -> Optional[torch.Tensor]:
        cfg, lw, l = self.cfg, self.layers[li], self.layer_start + li
        info, tr = batch.info, self.training
        sv = saved.full
        if sv is None:
            _, _, re = self._layer_forward(li, None, saved.h_in, batch, keep=True)
            sv = re.full
        elif "x1" not in sv:
            sv = dict(sv)
            sv["x1"] = ew.rmsnorm_fwd(saved.h_in, lw.ln1, cfg.rms_eps, want_rstd=False)[0]
            sv["x2"] = ew.rmsnorm_fwd(sv["h_mid"], lw.ln2, cfg.rms_eps, want_rstd=False)[0]
            if "gu" not in sv:
                # one GEMM rebuilds gate|up from x2 and the kept LoRA down-projection S'
                sv["gu"], s_new = lora_linear_forward(sv["x2"], lw.gate_up, self._stack(l, "gate_up"), info,
                                                      stream_id=self._sid(l, "gate_up"), training=tr, s=sv["s_gu"])
                if isinstance(s_new, list):  # unfused baseline: its stored masks were re-drawn
                    sv["s_gu"] = s_new
            sv["act"] = ew.swiglu_fwd(sv["gu"])
        d_act = lora_linear_backward(dh, sv["act"], sv["s_d"], lw.down, self._stack(l, "down"), info,
                                     stream_id=self._sid(l, "down"), training=tr)
        d_gu = ew.swiglu_bwd(d_act, sv["gu"])
        del d_act
        d_x2 = lora_linear_backward(d_gu, sv["x2"], sv["s_gu"], lw.gate_up, self._stack(l, "gate_up"), info,
                                    stream_id=self._sid(l, "gate_up"), training=tr)
        del d_gu
        dh_mid = ew.rmsnorm_bwd(d_x2, sv["h_mid"], lw.ln2, sv["rstd2"], dres=dh)
        d_attn = lora_linear_backward(dh_mid, sv["attn"], sv["s_o"], lw.o, self._stack(l, "o"), info,
                                      stream_id=self._sid(l, "o"), training=tr)
        d_qkv = att.attention_backward(sv["qkv"], sv["attn"], d_attn, sv["lse"], batch.attn_tiles,
                                       cfg.num_heads, cfg.num_kv_heads)
        ew.rope_inplace(d_qkv, batch.position_ids, self.cos, self.sin, cfg.num_heads + cfg.num_kv_heads,
                        cfg.head_dim, backward=True)
        d_x1 = lora_linear_backward(d_qkv, sv["x1"], sv["s_qkv"], lw.qkv, self._stack(l, "qkv"), info,
                                    stream_id=self._sid(l, "qkv"), need_dx=need_input_grad, training=tr)
        if not need_input_grad:
            return None
        return ew.rmsnorm_bwd(d_x1, saved.h_in, lw.ln1, sv["rstd1"], dres=dh_mid)

    # ------------------------------------------------------------------ activation memory plan
    def saved_bytes_per_layer(self, tokens: int) -> int:
        """Bytes a layer keeps between forward and backward in the "cheap" mode (GEMM and
        attention outputs; the elementwise results are rebuilt)."""
        c = self.cfg
        return tokens * (c.qkv_size + c.q_size + c.hidden_size + 2 * c.intermediate_size) * 2 \
            + c.num_heads * tokens * 4 + tokens * 4 * 256 * 2

    def working_set_bytes(self, tokens: int) -> int:
        """Transient device memory next to the kept activations, at its peak: the backward of
        a layer that re-runs gate|up (that output, the SwiGLU result, and both their gradients
        are alive around the SwiGLU backward), a handful of hidden-sized tensors, the q|k|v
        gradient, one chunk of logits of the loss head, and the bf16 scratch the NF4 weights are
        expanded into (allocated at the first use of each weight shape)."""
        c = self.cfg
        per_gu = tokens * 2 * c.intermediate_size * 2
        hidden = tokens * c.hidden_size * 2
        head = 2 * min(tokens, self.head_chunk_tokens) * c.vocab_size * 2 if self.is_last else 0
        scratch = 0
        if self.quantize:
            scratch = 2 * (c.qkv_size * c.hidden_size + c.hidden_size * c.q_size
                           + 3 * c.intermediate_size * c.hidden_size)
        return 3 * per_gu + 10 * hidden + 3 * tokens * c.qkv_size * 2 + head + scratch

    def _plan_modes(self, tokens: int) -> list:
        """Per-layer keep mode for the forward pass.  ``recompute=True`` -> all ``False``
        (recompute the layer from its input), ``False`` -> all ``True`` (keep everything),
        ``"auto"`` -> a memory plan over these levels, best value per byte first:

        * ``"nogu"``    keep the GEMM / attention outputs except gate|up (the backward re-runs
          that one GEMM plus two RMSNorms and SwiGLU): about half of the recomputation time
          for a third of the bytes;
        * ``"cheap"``   also keep gate|up on the device (only elementwise kernels are re-run);
        * ``"offload"`` like ``"cheap"``, with gate|up parked in pinned host memory;
        * ``False``     keep nothing but the layer input.

        As many layers as fit become ``"nogu"``.  The memory that is left keeps gate|up of the
        LAST layers on the device (their backward comes first, so nothing has to travel).  With
        offloading, gate|up of up to ``offload_max_layers`` of the remaining layers -- what the
        PCIe link drains during one forward pass, spread evenly so that the copies never pile
        up -- goes to host memory; only the rest re-runs the gate|up GEMM."""
        n = len(self.layers)
        if self.force_keep_modes is not None:
            return list(self.force_keep_modes)
        if self.recompute is True:
            return [False] * n
        if self.recompute is False:
            return [True] * n
        # One plan per stage, made for the largest microbatch seen (smaller ones just use less
        # memory): the plan must not change between microbatches, or host buffers would be
        # pinned in the middle of a step on some ranks and not on others.
        if self._modes_plan is None or tokens > self._modes_tokens:
            free, _ = torch.cuda.mem_get_info(self.device)
            free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
            per_full = self.saved_bytes_per_layer(tokens)
            per_gu = tokens * 2 * self.cfg.intermediate_size * 2
            per_part = per_full - per_gu
            h_in_all = n * tokens * self.cfg.hidden_size * 2
            budget = max(0, free - self.reserve_bytes - self.working_set_bytes(tokens) - h_in_all * self.max_inflight)
            budget //= self.max_inflight
            offload = self.offload_enabled and self.max_inflight == 1
            if offload:
                # copies still on their way out, and the ring of returning buffers unless it
                # exists already (then it is no longer part of the free memory)
                from .offload import ActivationOffloader as _AO

                budget = max(0, budget - (_AO.MAX_BACKLOG + (_AO.RING if self._offloader is None else 0)) * per_gu)
            n_part = int(min(n, budget // per_part))
            n_full = int(min(n_part, (budget - n_part * per_part) // per_gu))
            modes = [False] * (n - n_part) + ["nogu"] * (n_part - n_full) + ["cheap"] * n_full
            if offload:
                from .offload import default_host_budget_bytes, host_slot_bytes

                if self.offload_host_budget is None:  # fixed at the first plan: pinning shrinks MemAvailable
                    self.offload_host_budget = default_host_budget_bytes()
                cand = [li for li in range(n) if modes[li] == "nogu"]
                slots = int(self.offload_host_budget // host_slot_bytes(per_gu))
                # without a measured link rate: two layers out of three (a forward pass
                # produces gate|up about 1.5x faster than one PCIe 5 link drains it)
                cap = self.offload_max_layers if self.offload_max_layers is not None else (2 * n + 2) // 3
                take = max(0, min(len(cand), slots, cap))
                for j in range(take):  # evenly spread over the candidates
                    modes[cand[(j * len(cand)) // take]] = "offload"
            self._modes_plan, self._modes_tokens = modes, tokens
        return self._modes_plan

    def plan_activations(self, max_tokens: int) -> dict:
        """Make the activation plan now, for microbatches of up to ``max_tokens`` tokens, while
        no activations are alive (a plan made in the middle of a step sees less free memory)."""
        self._modes_plan = None
        self._plan_modes(max_tokens)
        return self.keep_summary(max_tokens)

    def set_offload(self, enabled: bool, host_budget_bytes: Optional[int] = None,
                    max_layers: Optional[int] = None) -> None:
        """Allow the memory plan to park gate|up outputs in pinned host memory (single
        microbatch in flight only).  Clears the cached plan."""
        self.offload_enabled = bool(enabled)
        self.offload_host_budget = host_budget_bytes
        self.offload_max_layers = max_layers
        self._modes_plan = None

    def prepare_offload(self, tokens: int, host_budget_bytes: Optional[int] = None,
                        max_layers: Optional[int] = None) -> bool:
        """Enable offloading for microbatches of up to ``tokens`` tokens and pin the host
        memory now.  ``max_layers`` = how many layers' gate|up the device-to-host link can take
        during one forward pass (measured link rate x forward time / bytes per layer).  Returns
        False (offloading left disabled) when the plan has nothing to park or the host refuses
        the pinned allocation."""
        self.set_offload(True, host_budget_bytes, max_layers)
        keys = [li for li, m in enumerate(self._plan_modes(tokens)) if m == "offload"]
        if keys:
            try:
                self._get_offloader(tokens).reserve_host(keys)
                return True
            except RuntimeError:
                pass
        self.disable_offload()
        return False

    def clear_plan(self) -> None:
        self._keep_plan = {}
        self._modes_plan = None

    def disable_offload(self) -> None:
        """Drop the offloader and give its pinned host buffers back to the operating system
        (the pinned-memory allocator would otherwise keep them cached)."""
        if self._offloader is not None:
            self._offloader.close()
        self._offloader = None
        self.set_offload(False)
        release = getattr(torch._C, "_host_emptyCache", None)
        if release is not None:
            try:
                release()
            except RuntimeError:
                pass  # only an optimisation: the buffers stay cached

    def _get_offloader(self, tokens: int):
        from .offload import ActivationOffloader

        numel = max(tokens, 1) * 2 * self.cfg.intermediate_size
        if self._offloader is None or self._offloader.slot_numel < numel:
            self._offloader = ActivationOffloader(self.device, numel)
        return self._offloader

    def keep_summary(self, tokens: int) -> dict:
        modes = self._plan_modes(tokens)
        if self._offloader is not None:
            self._offloader.reap()
        return {"keep_all_gemm_outputs": sum(m in (True, "cheap") for m in modes),
                "gate_up_in_host_memory": sum(m == "offload" for m in modes),
                "keep_all_but_gate_up": sum(m == "nogu" for m in modes),
                "recompute_layer": sum(m is False for m in modes)}

    def _plan_keep(self, tokens: int) -> int:
        """How many (trailing) layers keep their activations instead of recomputing them.
        ``recompute=True`` -> 0, ``False`` -> all, ``"auto"`` -> as many as fit in the free
        device memory after reserving room for one layer's working set, divided by the
        number of microbatches this stage holds in flight."""
        if self.recompute is True:
            return 0
        if self.recompute is False:
            return len(self.layers)
        key = (tokens,)
        if key not in self._keep_plan:
            free, _ = torch.cuda.mem_get_info(self.device)
            free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
            per = self.saved_bytes_per_layer(tokens)
            h_in_all = len(self.layers) * tokens * self.cfg.hidden_size * 2
            budget = free - self.reserve_bytes - 3 * per - h_in_all * self.max_inflight
            n = int(max(0, budget) // (per * self.max_inflight))
            self._keep_plan[key] = max(0, min(len(self.layers), n))
        return self._keep_plan[key]

    # ------------------------------------------------------------------ stage forward / backward
    def forward(self, batch: PackedBatch, h_in: Optional[torch.Tensor] = None):
        """Run this stage.  Returns ``(h_out, saved)``; on the last stage ``h_out`` is the
        pair ``(res, delta)`` that :meth:`loss_and_grad` consumes."""
        if self.is_first:
            delta = ew.embedding(batch.input_ids, self.embed)
            res = None
        else:
            delta, res = h_in, None
        saved = []
        modes = self._plan_modes(batch.num_tokens)
        for li in range(len(self.layers)):
            res, delta, sv = self._layer_forward(li, res, delta, batch, keep=modes[li])
            saved.append(sv)
        if self.is_last:
            return (res, delta), saved
        return ew.add(res, delta) if res is not None else delta, saved

    def loss_and_grad(self, out, batch: PackedBatch, loss_scale: float = 1.0):
        """Final norm + lm_head + cross-entropy, forward and backward together, in token
        chunks.  Returns ``(sum of token losses, d loss / d h)`` with the gradient already
        multiplied by ``loss_scale / num_loss_tokens``."""
        res, delta = out
        cfg = self.cfg
        x, h_fin, rstd = ew.rmsnorm_fwd(delta, self.final_norm, cfg.rms_eps, res=res)
        T = x.shape[0]
        n_loss = max(batch.num_loss_tokens, 1)
        dx = torch.empty_like(x)
        losses = torch.empty(T, dtype=torch.float32, device=x.device)
        chunk = self.head_chunk_tokens
        for t0 in range(0, T, chunk):
            t1 = min(T, t0 + chunk)
            logits = gemm_nt(x[t0:t1], self.lm_head)
            ew.cross_entropy_inplace(logits, batch.labels[t0:t1], loss_scale / n_loss, loss_out=losses[t0:t1])
            gemm_nn(logits, self.lm_head, out=dx[t0:t1])
            del logits
        dh = ew.rmsnorm_bwd(dx, h_fin, self.final_norm, rstd)
        return losses.sum(), dh

    def backward(self, saved: list, dh: torch.Tensor, batch: PackedBatch,
                 on_layer_done=None) -> Optional[torch.Tensor]:
        """Back-propagate ``dh`` (gradient w.r.t. this stage's output) through the layers;
        LoRA gradients accumulate in the arena.  Returns the gradient w.r.t. the stage input
        (``None`` on the first stage, whose input is the frozen embedding).
        ``on_layer_done(global layer index)`` is called right after the backward of each layer
        has been queued: from then on that layer's LoRA gradients of this microbatch are final."""
        # gate|up outputs parked in host memory come back two layers ahead of their use
        parked = [li for li in reversed(range(len(self.layers)))
                  if saved[li].full is not None and "gu_off" in saved[li].full]
        inflight: dict = {}

        def fetch_ahead():
            while parked and len(inflight) < max(1, len(self._offloader.ring) - 1):
                nxt = parked.pop(0)
                inflight[nxt] = self._offloader.prefetch(saved[nxt].full["gu_off"])

        fetch_ahead()
        for li in reversed(range(len(self.layers))):
            need = not (self.is_first and li == 0)
            slot = None
            if li in inflight:
                dev, ready, slot = inflight.pop(li)
                fetch_ahead()
                torch.cuda.current_stream(self.device).wait_event(ready)
                saved[li].full = dict(saved[li].full, gu=dev)
            dh = self._layer_backward(li, saved[li], dh, batch, need_input_grad=need)
            if slot is not None:
                self._offloader.release(slot)
            saved[li] = None
            if on_layer_done is not None:
                on_layer_done(self.layer_start + li)
        return dh

    def forward_backward(self, batch: PackedBatch, loss_scale: float = 1.0, on_layer_done=None) -> torch.Tensor:
        """Whole-model step for an unpartitioned model: returns the summed token loss."""
        if not (self.is_first and self.is_last):
            raise RuntimeError("forward_backward needs the whole model on this stage")
        out, saved = self.forward(batch)
        loss, dh = self.loss_and_grad(out, batch, loss_scale)
        del out
        self.backward(saved, dh, batch, on_layer_done=on_layer_done)
        return loss
