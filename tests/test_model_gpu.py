"""End-to-end engine checks on miniature decoders: loss and LoRA gradients against the fp32
autograd oracle, recomputation equivalence, NF4 base, and loss decrease under Adam."""

import pytest
import torch

from lorafusion_b200.models.config import AdapterSpec, get_model_config
from lorafusion_b200.models.decoder import DecoderStage
from lorafusion_b200.models.reference_model import reference_loss_and_grads
from lorafusion_b200.train.data import MicroBatchSpec, build_packed_batch
from lorafusion_b200.utils.testing import assert_close_two_rounds

pytestmark = pytest.mark.gpu


def _setup(model="tiny", quantize=False, recompute=True, dropout=0.1):
    cfg = get_model_config(model)
    adapters = [AdapterSpec("lora_0", r=16, lora_alpha=32, dropout=dropout),
                AdapterSpec("lora_1", r=8, lora_alpha=16, dropout=0.0)]
    stage = DecoderStage(cfg, adapters, "cuda", quantize=quantize, init_b_std=0.02, seed=3,
                         recompute=recompute)
    spec = MicroBatchSpec([(0, [100, 37, 200]), (1, [129, 64])])
    batch = build_packed_batch(spec, adapters, cfg.vocab_size, "cuda", seed=5)
    return stage, batch


@pytest.mark.parametrize("model,quantize", [("tiny", False), ("tiny-qwen", False), ("tiny", True)])
def test_engine_matches_autograd_oracle(model, quantize):
    stage, batch = _setup(model, quantize)
    loss = stage.forward_backward(batch)
    ref_loss, ref_grads = reference_loss_and_grads(stage, batch, device="cuda")
    assert abs(float(loss) - float(ref_loss)) / float(ref_loss) < 2e-2
    for key, (da_ref, db_ref) in ref_grads.items():
        st = stage.arena.stack(*key)
        assert_close_two_rounds(st.da, da_ref, atol=3e-2, rtol=5e-2, scale_atol_by_rms=True,
                                max_mismatch_ratio=5e-3, msg=f"dA {key}")
        assert_close_two_rounds(st.db, db_ref, atol=3e-2, rtol=5e-2, scale_atol_by_rms=True,
                                max_mismatch_ratio=5e-3, msg=f"dB {key}")


@pytest.mark.parametrize("mode", [False, "auto", "nogu", "offload"])
def test_recompute_is_bitwise_equivalent(mode):
    """Full recomputation, keeping everything, and the memory-planned mix (which keeps GEMM /
    attention outputs and rebuilds the elementwise ones) must give identical gradients."""
    s1, batch = _setup(recompute=True)
    s2, _ = _setup(recompute="auto" if mode in ("nogu", "offload") else mode)
    if mode == "nogu":  # first layer rebuilds gate|up from x2 and the kept S', second keeps it
        s2.force_keep_modes = ["nogu", "cheap"]
    if mode == "offload":  # gate|up of both layers travels to pinned host memory and back
        s2.force_keep_modes = ["offload", "offload"]
    l1 = s1.forward_backward(batch)
    l2 = s2.forward_backward(batch)
    assert float(l1) == float(l2)
    assert torch.equal(s1.arena.grad, s2.arena.grad)
    if mode == "offload":
        assert s2._offloader.bytes_out == 2 * batch.num_tokens * 2 * s2.cfg.intermediate_size * 2
        # a second microbatch reuses the host slots and ring buffers
        s1.arena.zero_grad(), s2.arena.zero_grad()
        assert float(s1.forward_backward(batch)) == float(s2.forward_backward(batch))
        assert torch.equal(s1.arena.grad, s2.arena.grad)
    if mode == "auto":
        assert s2._plan_keep(batch.num_tokens) == len(s2.layers)


def test_loss_decreases_with_adam():
    stage, batch = _setup(dropout=0.0)
    losses = []
    for _ in range(8):
        losses.append(float(stage.forward_backward(batch)) / batch.num_loss_tokens)
        for a in range(2):
            stage.arena.adam_step(a, lr=2e-3)
    assert losses[-1] < losses[0] - 0.05, losses
    assert float(stage.arena.grad.abs().max()) == 0.0


def test_pipeline_demo_chained_stages_match_whole_model():
    """Four stages run back to back on one GPU reproduce the unpartitioned model."""
    from lorafusion_b200.cli import pp_demo

    res = pp_demo.run("small", 4)
    assert res["layers_per_stage"] == [1, 1, 1, 1]
    assert abs(res["loss_whole"] - res["loss_chained"]) <= 1e-3 * abs(res["loss_whole"])
    assert res["max_rel_grad_diff"] < 2e-2
