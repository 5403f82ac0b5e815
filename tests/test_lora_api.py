"""Public fused-LoRA entry points: CPU oracle algebra (runs without a GPU) and, on a GPU,
the fused kernels against that oracle."""

import pytest
import torch

from lorafusion_b200.ops.batch_info import prepare_multi_lora_batch_info
from lorafusion_b200.ops.lora import fused_linear_lora, fused_linear_multi_lora
from lorafusion_b200.ops.philox import keep_mask
from lorafusion_b200.utils.testing import assert_close, assert_close_two_rounds


def _problem(M=2048, K=4096, N=4096, r=16, dtype=torch.float32, device="cpu", seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.02
    a = torch.randn(r, K, generator=g) * 0.02
    b = torch.randn(N, r, generator=g) * 0.02
    dy = torch.randn(M, N, generator=g)
    return [t.to(device=device, dtype=dtype) for t in (x, w, a, b, dy)]


def test_single_lora_cpu_oracle_matches_closed_form():
    """Single LoRA linear fwd+bwd on CPU fp32: X[2048,4096], W/A/B ~ N(0, 0.02), rank 16,
    alpha 32 (scaling 2), dropout 0.1 with seed 0; Y, dX, dA, dB against the closed-form
    expressions."""
    x, w, a, b, dy = _problem()
    scaling, p = 32 / 16, 0.1
    x.requires_grad_(True)
    a.requires_grad_(True)
    b.requires_grad_(True)
    y = fused_linear_lora(x, w, a, b, scaling, seed=0, dropout_p=p)
    y.backward(dy)
    keep = keep_mask(x.shape[0], x.shape[1], p, 0)
    xh = torch.where(keep, x.detach() / (1 - p), torch.zeros(()))
    s = xh @ a.detach().t()
    assert_close(y.detach(), x.detach() @ w.t() + scaling * s @ b.detach().t(), rtol=1e-4, atol=1e-4, msg="Y")
    ds = dy @ b.detach() * scaling
    assert_close(b.grad, scaling * dy.t() @ s, rtol=1e-4, atol=1e-3, msg="dB")
    assert_close(a.grad, ds.t() @ xh, rtol=1e-4, atol=1e-3, msg="dA")
    dx = dy @ w + torch.where(keep, (ds @ a.detach()) / (1 - p), torch.zeros(()))
    assert_close(x.grad, dx, rtol=1e-4, atol=1e-3, msg="dX")
    assert abs(float(keep.float().mean()) - 0.9) < 2e-3


def test_3d_and_2d_inputs_agree_on_cpu():
    x, w, a, b, _ = _problem(M=64, K=128, N=96, r=8)
    y2 = fused_linear_lora(x, w, a, b, 2.0, seed=3, dropout_p=0.0)
    y3 = fused_linear_lora(x.view(1, 64, 128), w, a, b, 2.0, seed=3, dropout_p=0.0)
    assert torch.equal(y2, y3.view(64, 96))


def test_batch_info_tables():
    info = prepare_multi_lora_batch_info([129, 130, 128], [0, 2, 1], [16, 32, 64], [0.1, 0.0, 0.1],
                                         [2.0, 1.0, 0.5], device="cpu")
    assert info.padded_seq_len_list == [256, 256, 128]
    assert info.block_to_lookup_table[:, 1].tolist() == [128, 1, 128, 2, 128]
    assert info.block_to_lookup_table[:, 0].tolist() == [16, 16, 32, 32, 64]
    assert info.block_to_lookup_table[:, 2].tolist() == [0, 0, 2, 2, 4]
    assert info.tile_adapter.tolist() == [0, 0, 2, 2, 1]
    assert info.segments == [(0, 0, 256), (2, 256, 512), (1, 512, 640)]
    assert info.adapter_scale.tolist() == [2.0, 0.5, 1.0]
    assert info.adapter_thresh16.tolist() == [6554, 6554, 0]
    assert info.enable_dropout and info.same_dropout_p_value is None
    assert info.max_r == 64 and info.num_active_adapters == 3


def _multi_problem(device, dtype, seg_lens=(300, 128, 257), ranks=(16, 32, 64), K=512, N=384):
    g = torch.Generator().manual_seed(5)
    padded = [((n + 127) // 128) * 128 for n in seg_lens]
    T = sum(padded)
    x = torch.randn(T, K, generator=g).to(device=device, dtype=dtype)
    w = (torch.randn(N, K, generator=g) * 0.03).to(device=device, dtype=dtype)
    a_list = [(torch.randn(r, K, generator=g) * 0.05).to(device=device, dtype=dtype) for r in ranks]
    b_list = [(torch.randn(N, r, generator=g) * 0.05).to(device=device, dtype=dtype) for r in ranks]
    dy = torch.randn(T, N, generator=g).to(device=device, dtype=dtype)
    return x, w, a_list, b_list, dy, padded


def test_multi_lora_cpu_oracle_segments():
    x, w, a_list, b_list, _, padded = _multi_problem("cpu", torch.float32)
    y = fused_linear_multi_lora(x, w, lora_a_list=a_list, lora_b_list=b_list, seq_len_list=[300, 128, 257],
                                lora_idx_list=[2, 0, 1], alpha_list=[1.0, 2.0, 0.5],
                                dropout_p_list=[0.0, 0.0, 0.0])
    start = 0
    for plen, a, alpha in zip(padded, [2, 0, 1], [1.0, 2.0, 0.5]):
        seg = x[start:start + plen]
        ref = seg @ w.t() + alpha * (seg @ a_list[a].t()) @ b_list[a].t()
        assert_close(y[start:start + plen], ref, rtol=1e-4, atol=1e-4, msg=f"segment at {start}")
        start += plen


@pytest.mark.gpu
@pytest.mark.parametrize("p", [0.0, 0.1])
def test_fused_linear_lora_gpu_matches_oracle(p):
    x, w, a, b, dy = _problem(dtype=torch.bfloat16, device="cuda", seed=1)
    leaves = [t.clone().requires_grad_(True) for t in (x, a, b)]
    y = fused_linear_lora(leaves[0].view(1, *x.shape), w, leaves[1], leaves[2], 2.0, seed=0, dropout_p=p)
    y.backward(dy.view(1, *dy.shape))
    ref_leaves = [t.float().cpu().requires_grad_(True) for t in (x, a, b)]
    y_ref = fused_linear_lora(ref_leaves[0], w.float().cpu(), ref_leaves[1], ref_leaves[2], 2.0, seed=0,
                              dropout_p=p)
    y_ref.backward(dy.float().cpu())
    assert_close_two_rounds(y.view(*dy.shape), y_ref.detach(), msg="Y")
    assert_close_two_rounds(leaves[0].grad, ref_leaves[0].grad, atol=1e-2, scale_atol_by_rms=True, msg="dX")
    assert_close_two_rounds(leaves[1].grad, ref_leaves[1].grad, atol=1e-2, rtol=3e-2, scale_atol_by_rms=True, msg="dA")
    assert_close_two_rounds(leaves[2].grad, ref_leaves[2].grad, atol=1e-2, rtol=3e-2, scale_atol_by_rms=True, msg="dB")


@pytest.mark.gpu
@pytest.mark.parametrize("mixed_p", [False, True])
def test_fused_linear_multi_lora_gpu_matches_oracle(mixed_p):
    x, w, a_list, b_list, dy, _ = _multi_problem("cuda", torch.bfloat16)
    kw = dict(seq_len_list=[300, 128, 257], lora_idx_list=[2, 0, 1], alpha_list=[1.0, 2.0, 0.5],
              dropout_p_list=[0.1, 0.0, 0.2] if mixed_p else [0.1, 0.1, 0.1], seed=11, stream_id=3)
    xg = x.clone().requires_grad_(True)
    ag = [t.clone().requires_grad_(True) for t in a_list]
    bg = [t.clone().requires_grad_(True) for t in b_list]
    y = fused_linear_multi_lora(xg.view(1, *x.shape), w, lora_a_list=ag, lora_b_list=bg, **kw)
    y.backward(dy.view(1, *dy.shape))
    xr = x.float().cpu().requires_grad_(True)
    ar = [t.float().cpu().requires_grad_(True) for t in a_list]
    br = [t.float().cpu().requires_grad_(True) for t in b_list]
    yr = fused_linear_multi_lora(xr, w.float().cpu(), lora_a_list=ar, lora_b_list=br, **kw)
    yr.backward(dy.float().cpu())
    assert_close_two_rounds(y.view(*dy.shape), yr.detach(), msg="Y")
    assert_close_two_rounds(xg.grad, xr.grad, atol=1e-2, scale_atol_by_rms=True, msg="dX")
    for i in range(3):
        assert_close_two_rounds(ag[i].grad, ar[i].grad, atol=1e-2, rtol=3e-2, scale_atol_by_rms=True, msg=f"dA[{i}]")
        assert_close_two_rounds(bg[i].grad, br[i].grad, atol=1e-2, rtol=3e-2, scale_atol_by_rms=True, msg=f"dB[{i}]")
