"""GPU numerics of the elementwise, NF4, cross-entropy, Adam and attention kernels against
plain fp32 PyTorch."""

import math

import pytest
import torch

from lorafusion_b200.utils.testing import assert_close, assert_close_two_rounds

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,H", [(7, 512), (130, 4096), (33, 8192)])
def test_rmsnorm(M, H):
    from lorafusion_b200.ops import elementwise as ew

    x, res, w = _rand(M, H, seed=1), _rand(M, H, seed=2), _rand(H, seed=3)
    dy, dres = _rand(M, H, seed=4), _rand(M, H, seed=5)
    y, h, rstd = ew.rmsnorm_fwd(x, w, 1e-5, res=res)
    hf = (x.float() + res.float()).to(torch.bfloat16).float().requires_grad_(True)
    var = hf.pow(2).mean(-1, keepdim=True)
    yf = hf * torch.rsqrt(var + 1e-5) * w.float()
    assert_close(h, (x.float() + res.float()).to(torch.bfloat16), msg="h")
    assert_close_two_rounds(y, yf.detach(), msg="rmsnorm y")
    yf.backward(dy.float())
    dx = ew.rmsnorm_bwd(dy, h, w, rstd, dres=dres)
    assert_close_two_rounds(dx, hf.grad + dres.float(), msg="rmsnorm dx")
    y2, h2, _ = ew.rmsnorm_fwd(x, w, 1e-5)
    assert h2 is x
    xf = x.float()
    assert_close_two_rounds(y2, xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float(),
                            msg="rmsnorm (no residual)")


def test_rope_roundtrip_and_values():
    from lorafusion_b200.ops import elementwise as ew

    M, Hq, Hkv, D = 300, 8, 2, 128
    qkv = _rand(M, (Hq + 2 * Hkv) * D, seed=6)
    pos = (torch.arange(M, device="cuda") % 97).int()
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(128, device="cuda").float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    ref = qkv.float().view(M, Hq + 2 * Hkv, D).clone()
    c, s = cos[pos.long()][:, None, :], sin[pos.long()][:, None, :]
    lo, hi = ref[:, : Hq + Hkv, : D // 2].clone(), ref[:, : Hq + Hkv, D // 2:].clone()
    ref[:, : Hq + Hkv, : D // 2] = lo * c - hi * s
    ref[:, : Hq + Hkv, D // 2:] = hi * c + lo * s
    work = qkv.clone()
    ew.rope_inplace(work, pos, cos, sin, Hq + Hkv, D)
    assert_close_two_rounds(work, ref.view(M, -1), msg="rope fwd")
    ew.rope_inplace(work, pos, cos, sin, Hq + Hkv, D, backward=True)
    assert_close_two_rounds(work, qkv.float(), atol=3e-2, msg="rope roundtrip")


def test_swiglu_embedding_add():
    from lorafusion_b200.ops import elementwise as ew

    M, I = 257, 1024
    gu, dout = _rand(M, 2 * I, seed=7), _rand(M, I, seed=8)
    g = gu[:, :I].float().requires_grad_(True)
    u = gu[:, I:].float().requires_grad_(True)
    ref = torch.nn.functional.silu(g) * u
    assert_close_two_rounds(ew.swiglu_fwd(gu), ref.detach(), msg="swiglu fwd")
    ref.backward(dout.float())
    assert_close_two_rounds(ew.swiglu_bwd(dout, gu), torch.cat([g.grad, u.grad], 1), msg="swiglu bwd")
    table = _rand(1000, 512, seed=9)
    ids = torch.randint(0, 1000, (77,), device="cuda", dtype=torch.int32)
    assert torch.equal(ew.embedding(ids, table), table[ids.long()])
    a, b = _rand(64, 256, seed=10), _rand(64, 256, seed=11)
    assert_close(ew.add(a, b), (a.float() + b.float()).to(torch.bfloat16), msg="add")


@pytest.mark.parametrize("V", [1000, 32000, 128256])
def test_cross_entropy(V):
    from lorafusion_b200.ops import elementwise as ew

    M = 50
    logits = _rand(M, V, scale=2.0, seed=12)
    labels = torch.randint(0, V, (M,), device="cuda", dtype=torch.int32)
    labels[::7] = -100
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, labels.long(), ignore_index=-100, reduction="none")
    n_valid = int((labels >= 0).sum())
    (ref.sum() / n_valid).backward()
    work = logits.clone()
    loss = ew.cross_entropy_inplace(work, labels, 1.0 / n_valid)
    assert_close(loss, ref.detach(), rtol=1e-3, atol=1e-3, msg="ce loss")
    assert_close_two_rounds(work, lf.grad, atol=1e-5, rtol=2e-2, msg="ce grad")


def test_adam_chunks_matches_torch():
    from lorafusion_b200.ops import elementwise as ew

    n = 5000
    torch.manual_seed(0)
    init = torch.randn(n, device="cuda")
    ref = init.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    # two regions: a flat one and a 2-D one where only columns [8, 24) of 32 are trainable;
    # the optimizer state is dense: 1000 elements, then the 100 x 16 window row by row
    # (a third region with odd offsets and sizes takes the kernel's scalar path)
    chunks = torch.tensor([[0, 1, 1000, 0, 1000, 0], [1024, 100, 32, 8, 16, 1000],
                           [4301, 10, 30, 3, 10, 2600]], dtype=torch.int64, device="cuda")
    trainable = torch.zeros(n, dtype=torch.bool, device="cuda")
    trainable[:1000] = True
    blk = torch.zeros(100, 32, dtype=torch.bool, device="cuda")
    blk[:, 8:24] = True
    trainable[1024:1024 + 3200] = blk.view(-1)
    blk3 = torch.zeros(10, 30, dtype=torch.bool, device="cuda")
    blk3[:, 3:13] = True
    trainable[4301:4601] = blk3.view(-1)

    def dense(t):
        return torch.cat([t[:1000], t[1024:4224].view(100, 32)[:, 8:24].reshape(-1),
                          t[4301:4601].view(10, 30)[:, 3:13].reshape(-1)])

    master = dense(init).clone()
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    work = init.to(torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        grad = g.clone()
        ref.grad = torch.where(trainable, g * 0.5, torch.zeros_like(g))
        opt.step()
        ew.adam_chunks(chunks, grad, master, m, v, work, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                       weight_decay=0.1, step=step, grad_scale=0.5)
        assert float(grad[:1000].abs().max()) == 0.0 and float(grad[1024:4224].abs().max()) == 0.0
        assert float(grad[4301:4601].abs().max()) == 0.0 and float(grad[4224:4301].abs().min()) > 0.0
    assert_close(master, dense(ref.detach()), rtol=1e-4, atol=1e-5, msg="adam master")
    assert_close(work[trainable], ref.detach()[trainable].to(torch.bfloat16), msg="adam bf16 copy")
    assert torch.equal(work[~trainable], init.to(torch.bfloat16)[~trainable])


@pytest.mark.parametrize("double_quant", [False, True])
def test_nf4_roundtrip(double_quant):
    from lorafusion_b200.ops import nf4

    w = _rand(256, 1024, scale=0.02, seed=13)
    q_gpu = nf4.quantize_nf4(w, double_quant=double_quant)
    q_cpu = nf4.quantize_nf4(w.cpu(), double_quant=double_quant)
    assert torch.equal(q_gpu.packed.cpu(), q_cpu.packed), "GPU and CPU quantisers disagree"
    deq = nf4.dequantize_nf4(q_gpu)
    ref = nf4.dequantize_nf4_reference(q_gpu, dtype=torch.float32)
    assert_close_two_rounds(deq, ref, atol=1e-4, msg="nf4 dequant")
    err = (deq.float() - w.float()).abs().max() / w.float().abs().max()
    assert float(err) < 0.2


def _attn_case(lens, Hq, Hkv, seed):
    from lorafusion_b200.ops import attention as att

    D = 128
    M = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    qkv = _rand(M, (Hq + 2 * Hkv) * D, scale=1.0, seed=seed).requires_grad_(True)
    tiles = att.build_attn_tiles(cu, "cuda")
    out = att.packed_attention(qkv, tiles, Hq, Hkv)
    d_out = _rand(M, Hq * D, seed=seed + 1)
    out.backward(d_out)
    qf = qkv.detach().float().requires_grad_(True)
    q = qf[:, : Hq * D].view(M, Hq, D)
    k = qf[:, Hq * D: (Hq + Hkv) * D].view(M, Hkv, D)
    v = qf[:, (Hq + Hkv) * D:].view(M, Hkv, D)
    ref = att.attention_reference(q, k, v, cu).view(M, Hq * D)
    ref.backward(d_out.float())
    return out, ref.detach(), qkv.grad, qf.grad


@pytest.mark.parametrize("lens,Hq,Hkv", [([128], 1, 1), ([256, 128], 2, 1), ([100, 37, 300, 129], 4, 2),
                                         ([1000, 24], 8, 1),
                                         # one query head per KV head and five key tiles: the three-stage K
                                         # ring and the two S buffers of dQ wrap around inside ONE head
                                         ([640], 2, 2),
                                         # five query heads per KV head (the 32B grouping), ragged lengths
                                         ([700, 513, 65], 10, 2)])
def test_attention_fwd_bwd(lens, Hq, Hkv):
    out, ref, dqkv, dref = _attn_case(lens, Hq, Hkv, seed=20)
    assert_close_two_rounds(out, ref, atol=2e-2, msg="attention fwd")
    D = 128
    assert_close_two_rounds(dqkv[:, : Hq * D], dref[:, : Hq * D], atol=5e-2, rtol=3e-2, msg="dQ")
    assert_close_two_rounds(dqkv[:, Hq * D: (Hq + Hkv) * D], dref[:, Hq * D: (Hq + Hkv) * D], atol=8e-2,
                            rtol=3e-2, msg="dK")
    assert_close_two_rounds(dqkv[:, (Hq + Hkv) * D:], dref[:, (Hq + Hkv) * D:], atol=8e-2, rtol=3e-2,
                            msg="dV")


def test_first_backward_of_a_process_may_be_a_custom_function():
    """A fresh process whose very first backward node is one of this package's autograd
    Functions: the autograd worker thread has made no CUDA runtime call yet, so no context is
    current in it when the backward builds its TMA tensor maps (a driver call).  The tensor-map
    helper binds the context of the device that owns the data and encodes again."""
    import subprocess
    import sys

    code = (
        "import torch\n"
        "from lorafusion_b200.ops import attention as att, _native\n"
        "from lorafusion_b200.ops import fused_linear_lora\n"
        "g = torch.Generator(device='cuda').manual_seed(0)\n"
        "qkv = torch.randn(128, 384, generator=g, device='cuda').to(torch.bfloat16).requires_grad_(True)\n"
        "tiles = att.build_attn_tiles([0, 128], 'cuda')\n"
        "out = att.packed_attention(qkv, tiles, 1, 1)\n"
        "out.backward(torch.ones_like(out))\n"
        "x = torch.randn(256, 512, generator=g, device='cuda').to(torch.bfloat16).requires_grad_(True)\n"
        "w = (torch.randn(512, 512, generator=g, device='cuda') * 0.03).to(torch.bfloat16)\n"
        "a = (torch.randn(16, 512, generator=g, device='cuda') * 0.03).to(torch.bfloat16).requires_grad_(True)\n"
        "b = (torch.randn(512, 16, generator=g, device='cuda') * 0.03).to(torch.bfloat16).requires_grad_(True)\n"
        "y = fused_linear_lora(x, w, a, b, alpha=2.0, dropout_p=0.1, seed=1)\n"
        "y.backward(torch.ones_like(y))\n"
        "torch.cuda.synchronize(); _native.check_device_errors()\n"
        "assert torch.isfinite(qkv.grad.float()).all() and torch.isfinite(x.grad.float()).all()\n"
        "print('first-backward ok')\n"
    )
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]   # the package is imported from the source tree
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=root)
    assert res.returncode == 0 and "first-backward ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
