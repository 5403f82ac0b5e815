"""nn.Module wrappers (LoRALinear, MultiLoRALinear, apply_lora, merge_qkv_proj) on CPU, where the
fused ops fall back to the plain-PyTorch oracle."""

import torch
from torch import nn

from lorafusion_b200.ops.batch_info import prepare_multi_lora_batch_info
from lorafusion_b200.ops.modules import (LoRALinear, MergedQKVLinear, MultiLoRALinear, apply_lora,
                                         merge_qkv_proj)


class _Attn(nn.Module):
    def __init__(self, h=64, kv=32):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(h, h), nn.Linear(h, kv), nn.Linear(h, kv)
        self.o_proj = nn.Linear(h, h, bias=False)


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = nn.ModuleList([nn.ModuleDict({"self_attn": _Attn()}) for _ in range(3)])
        self.lm_head = nn.Linear(64, 100, bias=False)


def test_lora_linear_matches_manual_math_and_trains_only_adapters():
    torch.manual_seed(0)
    base = nn.Linear(48, 40)
    m = LoRALinear(base, r=8, lora_alpha=16, lora_dropout=0.0)
    with torch.no_grad():
        m.lora_B.normal_(0, 0.1)
    x = torch.randn(2, 5, 48, requires_grad=True)
    y = m(x)
    ref = x @ base.weight.t() + base.bias + (x @ m.lora_A.t() @ m.lora_B.t()) * 2.0
    assert torch.allclose(y, ref, atol=1e-5)
    y.sum().backward()
    assert m.lora_A.grad is not None and m.lora_B.grad is not None and x.grad is not None
    assert not m.weight.requires_grad and m.weight.grad is None
    # dropout: eval mode is deterministic and equals the p = 0 result
    d = LoRALinear(base, r=8, lora_alpha=16, lora_dropout=0.5).eval()
    with torch.no_grad():
        d.lora_A.copy_(m.lora_A), d.lora_B.copy_(m.lora_B)
    assert torch.allclose(d(x), ref, atol=1e-5)
    d.train()
    assert not torch.allclose(d(x), ref, atol=1e-5)


def test_multi_lora_linear_per_segment_adapters():
    torch.manual_seed(1)
    base = nn.Linear(32, 24, bias=False)
    m = MultiLoRALinear(base, [(4, 8.0, 0.0), (8, 8.0, 0.0)]).eval()
    with torch.no_grad():
        for b in m.lora_B.values():
            b.normal_(0, 0.1)
    info = prepare_multi_lora_batch_info([100, 60], [1, 0], [8, 4], [0.0, 0.0], [1.0, 2.0], device="cpu")
    T = info.total_padded_tokens
    x = torch.randn(T, 32)
    m.set_batch_info(info)
    y = m(x)
    ref = x @ base.weight.t()
    # every row of a padded segment (128-row multiples) goes through the segment's adapter
    ref[:128] += (x[:128] @ m.lora_A["lora_1"].t() @ m.lora_B["lora_1"].t()) * 1.0
    ref[128:256] += (x[128:256] @ m.lora_A["lora_0"].t() @ m.lora_B["lora_0"].t()) * 2.0
    assert torch.allclose(y, ref, atol=1e-5)


def test_apply_lora_and_merge_qkv():
    torch.manual_seed(2)
    net = _Net()
    attn0 = net.layers[0]["self_attn"]
    x = torch.randn(7, 64)
    q, k, v = attn0.q_proj(x), attn0.k_proj(x), attn0.v_proj(x)
    n = merge_qkv_proj(net, layer_indices=[0, 2])
    assert n == 2 and isinstance(attn0.qkv_proj, MergedQKVLinear) and not hasattr(attn0, "q_proj")
    assert hasattr(net.layers[1]["self_attn"], "q_proj")
    q2, k2, v2 = attn0.qkv_proj.split(attn0.qkv_proj(x))
    assert torch.allclose(q, q2, atol=1e-6) and torch.allclose(k, k2, atol=1e-6) and torch.allclose(v, v2, atol=1e-6)
    back = attn0.qkv_proj.to_original()
    assert torch.allclose(back[1](x), k, atol=1e-6) and torch.allclose(back[2](x), v, atol=1e-6)
    apply_lora(net, r=4, lora_alpha=8, lora_dropout=0.0)
    assert isinstance(attn0.qkv_proj, LoRALinear) and isinstance(attn0.o_proj, LoRALinear)
    assert isinstance(net.lm_head, nn.Linear)  # not a target
    trainable = [n_ for n_, p in net.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n_ for n_ in trainable)
    streams = {m.stream_id for m in net.modules() if isinstance(m, LoRALinear)}
    assert len(streams) == sum(isinstance(m, LoRALinear) for m in net.modules())
