"""Plain PyTorch (fp32, autograd) evaluation of the same decoder, used as the oracle for the
hand-written engine on miniature models.  It reads the frozen weights and the adapters out of
a :class:`DecoderStage`, so both paths see identical parameters."""

from __future__ import annotations

import torch

from ..ops.attention import attention_reference
from ..ops.nf4 import NF4Weight, dequantize_nf4_reference
from ..ops.philox import keep_mask
from .decoder import DecoderStage, PackedBatch


def _dense(w) -> torch.Tensor:
    return (dequantize_nf4_reference(w, torch.float32) if isinstance(w, NF4Weight) else w.float())


def reference_loss_and_grads(stage: DecoderStage, batch: PackedBatch, device="cpu"):
    """Returns ``(summed token loss, {(layer, proj): (dA [n, R, K], dB [n, N, R])})`` computed
    with autograd in fp32.  Gradients are scaled by ``1 / num_loss_tokens`` like the engine."""
    cfg = stage.cfg
    dev = torch.device(device)
    info = batch.info
    T = batch.num_tokens
    ids = batch.input_ids.long().to(dev)
    labels = batch.labels.long().to(dev)
    pos = batch.position_ids.long().to(dev)
    cos, sin = stage.cos.to(dev)[pos], stage.sin.to(dev)[pos]
    row_adapter = info.tile_adapter.long().to(dev).repeat_interleave(128)[:T]
    n_ad = stage.arena.num_adapters if stage.arena is not None else 0
    leaves = {}

    def rms(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float().to(dev)

    def lora_linear(x, w, key, bias=None):
        y = x @ _dense(w).to(dev).t()
        if bias is not None:
            y = y + bias.float().to(dev)
        if stage.arena is None:
            return y
        st = stage.arena.stack(*key)
        a = st.a.float().to(dev).clone().requires_grad_(True)
        b = st.b.float().to(dev).clone().requires_grad_(True)
        leaves[key] = (a, b)
        sid = stage._sid(*key)
        add = torch.zeros_like(y)
        for i in range(n_ad):
            rows = row_adapter == i
            if not bool(rows.any()):
                continue
            spec = stage.adapters[i]
            xi = x[rows]
            if stage.training and spec.dropout > 0:
                km = keep_mask(T, x.shape[1], spec.dropout, info.seed, sid).to(dev)[rows]
                xi = torch.where(km, xi / (1 - spec.dropout), torch.zeros((), device=dev))
            add[rows] = (xi @ a[i].t()) @ b[i].t() * spec.scaling
        return y + add

    h = stage.embed.float().to(dev)[ids]
    for li, lw in enumerate(stage.layers):
        l = stage.layer_start + li
        x1 = rms(h, lw.ln1, cfg.rms_eps)
        qkv = lora_linear(x1, lw.qkv, (l, "qkv"), lw.qkv_bias)
        q = qkv[:, :cfg.q_size].view(T, cfg.num_heads, cfg.head_dim)
        k = qkv[:, cfg.q_size:cfg.q_size + cfg.kv_size].view(T, cfg.num_kv_heads, cfg.head_dim)
        v = qkv[:, cfg.q_size + cfg.kv_size:].view(T, cfg.num_kv_heads, cfg.head_dim)

        def rot(t):
            half = cfg.head_dim // 2
            lo, hi = t[..., :half], t[..., half:]
            c, s = cos[:, None, :], sin[:, None, :]
            return torch.cat([lo * c - hi * s, hi * c + lo * s], -1)

        attn = attention_reference(rot(q), rot(k), v, batch.cu_seqlens).view(T, cfg.q_size)
        h = h + lora_linear(attn, lw.o, (l, "o"))
        x2 = rms(h, lw.ln2, cfg.rms_eps)
        gu = lora_linear(x2, lw.gate_up, (l, "gate_up"))
        i_sz = cfg.intermediate_size
        act = torch.nn.functional.silu(gu[:, :i_sz]) * gu[:, i_sz:]
        h = h + lora_linear(act, lw.down, (l, "down"))
    x = rms(h, stage.final_norm, cfg.rms_eps)
    logits = x @ stage.lm_head.float().to(dev).t()
    loss = torch.nn.functional.cross_entropy(logits, labels, ignore_index=-100, reduction="sum")
    (loss / max(batch.num_loss_tokens, 1)).backward()
    grads = {k: (a.grad, b.grad) for k, (a, b) in leaves.items()}
    return loss.detach(), grads
