"""Tensor-parallel (+ sequence-parallel) decoder stage.

The reference runs with tensor parallelism fixed to 1
(``benchmarks_paper/bench_multi_gpu.py:624``); the 32B (TP2 x PP4) and 70B (TP4 x PP2)
configurations need it.  Layout, Megatron style:

* q|k|v and gate|up are **column-parallel** (each rank owns ``heads / tp`` heads and
  ``intermediate / tp`` channels); o and down are **row-parallel**.
* between blocks the residual stream is **sequence-parallel**: each rank holds ``T / tp``
  token rows, so RMSNorm, the residual adds, the embedding and the loss run on a token shard.
* the collectives live inside the GEMM kernels (``parallel/tp_ops.py``): column-parallel
  forward = all-gather -> GEMM, row-parallel forward = GEMM -> reduce-scatter, and mirrored
  in the backward (dX of column-parallel = GEMM -> reduce-scatter, dX of row-parallel =
  all-gather(dY) -> GEMM).
* LoRA: ``A`` of column-parallel and ``B`` of row-parallel projections are replicated, the
  other factor is sharded with the base weight.  The down-projection ``S' = drop(x) A^T`` of a
  column-parallel layer is computed on the token shard and all-gathered together with ``x``;
  for a row-parallel layer every rank adds its partial ``S'_p B^T`` to its partial output
  (linearity).  Gradients of replicated factors are partial sums per rank and are summed over
  the TP group right before the optimizer step (``reduce_replicated_grads``).
"""

from __future__ import annotations

from dataclasses import replace
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import attention as att
from ..ops import elementwise as ew
from ..ops import lora_kernels as lk
from ..ops.gemm import gemm_nn, gemm_nt
from ..ops.lora import materialize_weight
from ..ops.nf4 import NF4Weight, quantize_nf4
from ..parallel.tp_ops import TpContext, ag_gemm, gemm_rs
from .adapters import LoRAArena
from .config import AdapterSpec, ModelConfig
from .decoder import DecoderStage, LayerSaved, LayerWeights, PackedBatch

TILE = 128


def local_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    if cfg.num_heads % tp or cfg.num_kv_heads % tp or cfg.intermediate_size % (tp * 256):
        raise ValueError(f"{cfg.name}: heads / kv heads / intermediate size are not divisible by tp={tp}")
    return replace(cfg, name=f"{cfg.name}-tp{tp}", num_heads=cfg.num_heads // tp,
                   num_kv_heads=cfg.num_kv_heads // tp, intermediate_size=cfg.intermediate_size // tp)


def _shard_rows(w: torch.Tensor, parts: Sequence[int], rank: int, tp: int) -> torch.Tensor:
    """Row shard of a weight made of stacked blocks (q|k|v or gate|up): every block is cut in
    ``tp`` equal row slices and slice ``rank`` of each block is kept."""
    out, r0 = [], 0
    for n in parts:
        step = n // tp
        out.append(w[r0 + rank * step:r0 + (rank + 1) * step])
        r0 += n
    return torch.cat(out, 0).contiguous()


class TpDecoderStage(DecoderStage):
    """A :class:`DecoderStage` whose layers are split over a tensor-parallel group.  Built
    from the *global* config; all shapes inside are the rank-local ones."""

    def __init__(self, cfg: ModelConfig, adapters: Sequence[AdapterSpec], device, tp_group, *,
                 max_tokens: int, **kw):
        self.tp_group = tp_group
        self.tp = dist.get_world_size(tp_group) if (dist.is_initialized() and tp_group is not None) else 1
        self.tp_rank = dist.get_rank(tp_group) if self.tp > 1 else 0
        self.global_cfg = cfg
        super().__init__(local_config(cfg, self.tp), adapters, device, **kw)
        c = self.cfg
        self.ctx = TpContext(tp_group, device, max_tokens=max_tokens,
                             max_features=max(c.hidden_size, c.qkv_size, 2 * c.intermediate_size))

    # ------------------------------------------------------------------ construction from a full model
    @classmethod
    def from_full(cls, full: DecoderStage, tp_group, *, max_tokens: int, quantize: Optional[bool] = None,
                  recompute=True) -> "TpDecoderStage":
        """Shard an unpartitioned stage (weights and adapters) for this rank: the result
        computes exactly what ``full`` computes, split over the TP group."""
        cfg = full.cfg
        quantize = full.quantize if quantize is None else quantize
        self = cls(cfg, full.adapters, full.device, tp_group, max_tokens=max_tokens,
                   layer_start=full.layer_start, layer_end=full.layer_end, quantize=False, recompute=recompute,
                   init_b_std=0.0, seed=0)
        r, tp = self.tp_rank, self.tp
        i_full = cfg.intermediate_size

        def maybe_q(w):
            return quantize_nf4(w) if quantize else w

        for li, lw in enumerate(full.layers):
            dense = {k: materialize_weight(getattr(lw, k)).clone() for k in ("qkv", "o", "gate_up", "down")}
            q_loc, i_loc = cfg.q_size // tp, i_full // tp
            self.layers[li] = LayerWeights(
                ln1=lw.ln1.clone(), ln2=lw.ln2.clone(),
                qkv=maybe_q(_shard_rows(dense["qkv"], [cfg.q_size, cfg.kv_size, cfg.kv_size], r, tp)),
                o=maybe_q(dense["o"][:, r * q_loc:(r + 1) * q_loc].contiguous()),
                gate_up=maybe_q(_shard_rows(dense["gate_up"], [i_full, i_full], r, tp)),
                down=maybe_q(dense["down"][:, r * i_loc:(r + 1) * i_loc].contiguous()),
                qkv_bias=None if lw.qkv_bias is None else _shard_rows(
                    lw.qkv_bias[:, None], [cfg.q_size, cfg.kv_size, cfg.kv_size], r, tp)[:, 0].contiguous())
        self.embed = None if full.embed is None else full.embed.clone()
        self.lm_head = None if full.lm_head is None else full.lm_head.clone()
        self.final_norm = None if full.final_norm is None else full.final_norm.clone()
        if full.arena is not None:
            n = full.arena.num_adapters
            for (l, proj), fv in full.arena.views.items():
                lv = self.arena.views[(l, proj)]
                for name in ("work",):  # padded layout; the dense fp32 master follows below
                    src, dst = getattr(full.arena, name), getattr(self.arena, name)
                    fa = src[fv.a_offset:fv.a_offset + n * fv.R * fv.K].view(n, fv.R, fv.K)
                    fb = src[fv.b_offset:fv.b_offset + n * fv.N * fv.R].view(n, fv.N, fv.R)
                    la = dst[lv.a_offset:lv.a_offset + n * lv.R * lv.K].view(n, lv.R, lv.K)
                    lb = dst[lv.b_offset:lv.b_offset + n * lv.N * lv.R].view(n, lv.N, lv.R)
                    if proj in ("qkv", "gate_up"):      # A replicated, B row-sharded per block
                        la.copy_(fa)
                        parts = [s for _, s in fv.subs]
                        for a_i in range(n):
                            lb[a_i].copy_(_shard_rows(fb[a_i], parts, r, tp))
                    else:                                # A column-sharded, B replicated
                        step = fv.K // tp
                        la.copy_(fa[:, :, r * step:(r + 1) * step])
                        lb.copy_(fb)
            self.arena.sync_master_from_work()
        return self

    # ------------------------------------------------------------------ activation memory plan
    def saved_bytes_per_layer(self, tokens: int, mode="cheap") -> int:
        """Bytes one layer keeps on THIS rank: column-sharded GEMM outputs over all tokens, the
        token-sharded residual stream, and (mode True) the tensors "cheap" rebuilds instead."""
        c, tp = self.cfg, self.tp   # c holds the rank-local sizes
        ts = tokens // tp
        kept = tokens * (c.qkv_size + c.q_size + 2 * c.intermediate_size) * 2 + ts * c.hidden_size * 2 \
            + c.num_heads * tokens * 4 + tokens * 4 * 256 * 2
        if mode is True:
            kept += 2 * ts * c.hidden_size * 2 + tokens * c.intermediate_size * 2
        return kept

    def _plan_modes(self, tokens: int) -> list:
        """Per-layer keep mode: ``True`` (keep everything), ``"cheap"`` (keep GEMM / attention
        outputs, rebuild the normalised inputs and the SwiGLU output with elementwise kernels) or
        ``False`` (recompute the layer, which repeats its collectives).  With ``recompute="auto"``
        as many trailing layers as fit become ``"cheap"``; the tensor-parallel ranks agree on the
        smallest count any of them can afford, since a recomputed layer runs fused collectives
        that every rank must enter."""
        n = len(self.layers)
        if self.force_keep_modes is not None:
            return list(self.force_keep_modes)
        if self.recompute is True:
            return [False] * n
        if self.recompute is False:
            return [True] * n
        if self._modes_plan is None or tokens > self._modes_tokens:
            free, _ = torch.cuda.mem_get_info(self.device)
            free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
            ts = tokens // self.tp
            h_in_all = n * ts * self.cfg.hidden_size * 2
            budget = free - self.reserve_bytes - self.working_set_bytes(tokens) - h_in_all * self.max_inflight
            n_keep = int(max(0, budget) // (self.saved_bytes_per_layer(tokens) * self.max_inflight))
            n_keep = max(0, min(n, n_keep))
            if self.tp > 1:
                t = torch.tensor([n_keep], dtype=torch.int64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.tp_group)
                n_keep = int(t.item())
            self._modes_plan, self._modes_tokens = [False] * (n - n_keep) + ["cheap"] * n_keep, tokens
        return self._modes_plan

    # ------------------------------------------------------------------ helpers
    def _shard(self, t: torch.Tensor) -> torch.Tensor:
        ms = t.shape[0] // self.tp
        return t[self.tp_rank * ms:(self.tp_rank + 1) * ms]

    def _shard_info(self, batch: PackedBatch):
        """Tile-adapter table and segment table of this rank's token rows."""
        info = batch.info
        T = batch.num_tokens
        ms = T // self.tp
        r0, r1 = self.tp_rank * ms, (self.tp_rank + 1) * ms
        key = ("tp_shard", self.tp_rank, self.tp)
        cache = info.__dict__.setdefault("_tp_cache", {})
        if key not in cache:
            segs = []
            for a, s, e in info.segments:
                lo, hi = max(s, r0), min(e, r1)
                if hi > lo:
                    segs.append((a, lo - r0, hi - r0))
            cache[key] = (info.tile_adapter[r0 // TILE:r1 // TILE], lk.SegmentTable(segs, self.device, total_rows=ms))
        return cache[key]

    def _drop(self, info, sid: int, *, row_offset: int = 0, col_offset: int = 0):
        d = info.dropout_spec(sid, self.training)
        if d.active:
            d = replace(d, row_offset=row_offset, col_offset=col_offset)
        return d

    # ------------------------------------------------------------------ one layer
    def _layer_forward(self, li: int, res, delta, batch: PackedBatch, keep):
        cfg, lw, l, ctx = self.cfg, self.layers[li], self.layer_start + li, self.ctx
        info, T, r = batch.info, batch.num_tokens, self.tp_rank
        ms = T // self.tp
        ta_shard, _ = self._shard_info(batch)
        H = cfg.hidden_size
        q_loc, i_loc = cfg.q_size, cfg.intermediate_size  # local sizes (cfg is the local config)
        st = {p: self._stack(l, p) for p in ("qkv", "o", "gate_up", "down")}

        def col_parallel(x_in, res_in, ln, proj, w, bias=None):
            """rmsnorm (token shard) -> [x | S'] all-gather -> fused GEMM.  Returns
            (y_local [T, N_local], x_shard, h_shard, rstd, s_full copy)."""
            x_sh, h_sh, rstd = ew.rmsnorm_fwd(x_in, ln, cfg.rms_eps, res=res_in, out=ctx.own_gather_rows(T, H))
            stack = st[proj]
            R = stack.a.shape[1]
            lk.lora_down(x_sh, stack.a, tile_adapter=ta_shard, adapter_scale=info.adapter_scale,
                         dropout=self._drop(info, self._sid(l, proj), row_offset=r * ms),
                         out=ctx.own_gather2_rows(T, R))
            y = ag_gemm(ctx, T, H, materialize_weight(w, T), slab_cols=R, b2=stack.b, b2_adapter_rows=stack.b.shape[1],
                        tile_adapter=info.tile_adapter, bias=bias)
            # (the normalised shard lives in the gather buffer: copy it out only if the backward will want it)
            return y, (x_sh.clone() if keep is True else None), h_sh, rstd, ctx.gather2_view(T, R).clone()

        def row_parallel(x_loc, proj, w, k_loc, residual=None):
            stack = st[proj]
            s_p = lk.lora_down(x_loc, stack.a, tile_adapter=info.tile_adapter, adapter_scale=info.adapter_scale,
                               dropout=self._drop(info, self._sid(l, proj), col_offset=r * k_loc))
            y_sh = gemm_rs(ctx, x_loc, materialize_weight(w, T), s=s_p, b2=stack.b, b2_adapter_rows=stack.b.shape[1],
                           tile_adapter=info.tile_adapter, residual=residual)
            return y_sh, s_p

        qkv, x1, h_in, rstd1, s_qkv = col_parallel(delta, res, lw.ln1, "qkv", lw.qkv, lw.qkv_bias)
        ew.rope_inplace(qkv, batch.position_ids, self.cos, self.sin, cfg.num_heads + cfg.num_kv_heads, cfg.head_dim)
        attn, lse = att.attention_forward(qkv, batch.attn_tiles, cfg.num_heads, cfg.num_kv_heads)
        o, s_o = row_parallel(attn, "o", lw.o, q_loc)
        gu, x2, h_mid, rstd2, s_gu = col_parallel(o, h_in, lw.ln2, "gate_up", lw.gate_up)
        act = ew.swiglu_fwd(gu)
        d, s_d = row_parallel(act, "down", lw.down, i_loc)
        full = None
        if keep:
            full = dict(rstd1=rstd1, qkv=qkv, attn=attn, lse=lse, s_qkv=s_qkv, s_o=s_o, h_mid=h_mid,
                        rstd2=rstd2, gu=gu, s_gu=s_gu, s_d=s_d)
            if keep is True:  # "cheap" drops what one elementwise kernel rebuilds from kept tensors
                full.update(x1=x1, x2=x2, act=act)
        return h_mid, d, LayerSaved(h_in, full)

    def _layer_backward(self, li: int, saved: LayerSaved, dh, batch: PackedBatch, need_input_grad: bool = True):
        cfg, lw, l, ctx = self.cfg, self.layers[li], self.layer_start + li, self.ctx
        info, T, r = batch.info, batch.num_tokens, self.tp_rank
        ms = T // self.tp
        ta_shard, segs_shard = self._shard_info(batch)
        H = cfg.hidden_size
        q_loc, i_loc = cfg.q_size, cfg.intermediate_size
        st = {p: self._stack(l, p) for p in ("qkv", "o", "gate_up", "down")}
        sv = saved.full
        if sv is None:
            _, _, re = self._layer_forward(li, None, saved.h_in, batch, keep=True)
            sv = re.full
        elif "x1" not in sv:  # "cheap": the normalised token shards and the SwiGLU output are rebuilt
            sv = dict(sv)
            sv["x1"] = ew.rmsnorm_fwd(saved.h_in, lw.ln1, cfg.rms_eps, want_rstd=False)[0]
            sv["x2"] = ew.rmsnorm_fwd(sv["h_mid"], lw.ln2, cfg.rms_eps, want_rstd=False)[0]
            sv["act"] = ew.swiglu_fwd(sv["gu"])

        def row_parallel_bwd(dy_sh, x_loc, s_p, proj, w, k_loc):
            """all-gather(dY | dS) -> dX_local = dY_full W_shard + keep (.) (dS_full A_shard)."""
            stack = st[proj]
            R = stack.a.shape[1]
            ctx.own_gather_rows(T, H).copy_(dy_sh)
            lk.lora_ds(dy_sh, stack.b, tile_adapter=ta_shard, adapter_scale=info.adapter_scale,
                       out=ctx.own_gather2_rows(T, R))
            drop = self._drop(info, self._sid(l, proj), col_offset=r * k_loc)
            dx_loc = ag_gemm(ctx, T, H, materialize_weight(w, T), w_mn=True, slab_cols=R, b2=stack.a,
                             b2_adapter_rows=R, tile_adapter=info.tile_adapter,
                             dropout_kwargs=drop.kwargs() if drop.active else None)
            dy_full, ds_full = ctx.gather_view(T, H), ctx.gather2_view(T, R)
            lk.lora_db(dy_full, s_p, info.segment_table, stack.db)        # partial: summed over TP later
            lk.lora_da(x_loc, ds_full, info.segment_table, stack.da, dropout=drop)
            return dx_loc

        def col_parallel_bwd(dy_loc, x_sh, s_full, proj, w, need_dx=True):
            """dX_shard = reduce_scatter(dY_local W_shard + keep (.) (dS_p A)); dS reduced over TP
            for the replicated A's gradient."""
            stack = st[proj]
            ds_p = lk.lora_ds(dy_loc, stack.b, tile_adapter=info.tile_adapter, adapter_scale=info.adapter_scale)
            lk.lora_db(dy_loc, s_full, info.segment_table, stack.db)
            ds_f32 = ds_p.float()
            ds_sh = torch.empty((ms, ds_p.shape[1]), dtype=torch.float32, device=self.device)
            if self.tp > 1:
                dist.reduce_scatter_tensor(ds_sh, ds_f32, group=self.tp_group)
            else:
                ds_sh.copy_(ds_f32)
            drop_sh = self._drop(info, self._sid(l, proj), row_offset=r * ms)
            lk.lora_da(x_sh, ds_sh.to(torch.bfloat16), segs_shard, stack.da, dropout=drop_sh)  # partial over TP
            if not need_dx:
                return None
            drop = self._drop(info, self._sid(l, proj))
            return gemm_rs(ctx, dy_loc, materialize_weight(w, T), w_mn=True, s=ds_p, b2=stack.a,
                           b2_adapter_rows=stack.a.shape[1], tile_adapter=info.tile_adapter,
                           dropout_kwargs=drop.kwargs() if drop.active else None)

        d_act = row_parallel_bwd(dh, sv["act"], sv["s_d"], "down", lw.down, i_loc)
        d_gu = ew.swiglu_bwd(d_act, sv["gu"])
        d_x2 = col_parallel_bwd(d_gu, sv["x2"], sv["s_gu"], "gate_up", lw.gate_up)
        dh_mid = ew.rmsnorm_bwd(d_x2, sv["h_mid"], lw.ln2, sv["rstd2"], dres=dh)
        d_attn = row_parallel_bwd(dh_mid, sv["attn"], sv["s_o"], "o", lw.o, q_loc)
        d_qkv = att.attention_backward(sv["qkv"], sv["attn"], d_attn, sv["lse"], batch.attn_tiles, cfg.num_heads,
                                       cfg.num_kv_heads)
        ew.rope_inplace(d_qkv, batch.position_ids, self.cos, self.sin, cfg.num_heads + cfg.num_kv_heads,
                        cfg.head_dim, backward=True)
        d_x1 = col_parallel_bwd(d_qkv, sv["x1"], sv["s_qkv"], "qkv", lw.qkv, need_dx=need_input_grad)
        if not need_input_grad:
            return None
        return ew.rmsnorm_bwd(d_x1, saved.h_in, lw.ln1, sv["rstd1"], dres=dh_mid)

    # ------------------------------------------------------------------ stage forward / loss (token shards)
    def forward(self, batch: PackedBatch, h_in: Optional[torch.Tensor] = None):
        """``h_in`` / the returned activation are this rank's token shard ``[T / tp, H]``."""
        if self.is_first:
            delta = ew.embedding(self._shard(batch.input_ids).contiguous(), self.embed)
        else:
            delta = h_in
        res, saved = None, []
        modes = self._plan_modes(batch.num_tokens)
        for li in range(len(self.layers)):
            res, delta, sv = self._layer_forward(li, res, delta, batch, keep=modes[li])
            saved.append(sv)
        if self.is_last:
            return (res, delta), saved
        return ew.add(res, delta) if res is not None else delta, saved

    def loss_and_grad(self, out, batch: PackedBatch, loss_scale: float = 1.0):
        res, delta = out
        cfg = self.cfg
        x, h_fin, rstd = ew.rmsnorm_fwd(delta, self.final_norm, cfg.rms_eps, res=res)
        labels = self._shard(batch.labels).contiguous()
        Ts = x.shape[0]
        n_loss = max(batch.num_loss_tokens, 1)
        dx = torch.empty_like(x)
        losses = torch.empty(Ts, dtype=torch.float32, device=x.device)
        for t0 in range(0, Ts, self.head_chunk_tokens):
            t1 = min(Ts, t0 + self.head_chunk_tokens)
            logits = gemm_nt(x[t0:t1], self.lm_head)
            ew.cross_entropy_inplace(logits, labels[t0:t1], loss_scale / n_loss, loss_out=losses[t0:t1])
            gemm_nn(logits, self.lm_head, out=dx[t0:t1])
        loss = losses.sum()
        if self.tp > 1:
            dist.all_reduce(loss, group=self.tp_group)
        return loss, ew.rmsnorm_bwd(dx, h_fin, self.final_norm, rstd)

    # ------------------------------------------------------------------ replicated-factor gradients
    def replicated_grad_views(self, adapter: Optional[int] = None, layers: Optional[tuple] = None) -> list:
        """fp32 gradient tensors that are partial sums per TP rank: A of column-parallel and
        B of row-parallel projections (of one adapter, or of all; of layers ``lo <= l < hi``, or
        of all)."""
        out = []
        for (l, proj), v in self.arena.views.items():
            if layers is not None and not (layers[0] <= l < layers[1]):
                continue
            g = v.stack.da if proj in ("qkv", "gate_up") else v.stack.db
            out.append(g if adapter is None else g[adapter])
        return out

    def reduce_replicated_grads(self, adapter: Optional[int] = None, layers: Optional[tuple] = None) -> None:
        """Sum the partial gradients of replicated LoRA factors over the TP group (call right
        before the optimizer step of ``adapter``; ``None`` = every adapter; ``layers`` limits
        it to a group of layers so that it can run while the backward is still below them)."""
        if self.tp <= 1 or self.arena is None:
            return
        views = self.replicated_grad_views(adapter, layers)
        if not views:
            return
        flat = torch.cat([v.reshape(-1) for v in views])
        dist.all_reduce(flat, group=self.tp_group)
        off = 0
        for v in views:
            n = v.numel()
            v.copy_(flat[off:off + n].view_as(v))
            off += n
