"""Analytic predictor: interpolation, collective model, memory feasibility, enumeration (CPU)."""

import pytest

from lorafusion_b200.simulator import predictor as P


def test_collective_model_accepts_both_spellings_and_scales():
    hw = P.HardwareSpec()
    a = P.collective_time_ms("all-reduce", 1 << 30, 8, hw)
    b = P.collective_time_ms("allreduce", 1 << 30, 8, hw)
    assert a == b and 2.0 < a < 4.0          # 2*(7/8) GiB at ~725 GB/s
    assert P.collective_time_ms("allgather", 1 << 20, 1, hw) == 0.0
    with pytest.raises(ValueError):
        P.collective_time_ms("broadcast", 1, 2, hw)
    assert P.overlap_time(10.0, 4.0, 1.0) == 10.0 and P.overlap_time(10.0, 4.0, 0.0) == 14.0


def test_profile_roundtrip_and_interpolation(tmp_path):
    prof = P.synthesize_profile("llama-3.1-8b")
    assert prof.lora_params_per_layer_per_adapter == 1310720   # r=16 on all 7 linears of an 8B layer
    prof.save(tmp_path / "8b.yaml")
    back = P.LoRALLMProfileResult.load(tmp_path / "8b.yaml")
    assert back == prof
    assert prof.layer_fwd(4096) < prof.layer_fwd(6000) < prof.layer_fwd(8192)
    assert abs(prof.layer_fwd(32768) - 2 * prof.layer_fwd(16384)) < 1e-9


def test_70b_memory_and_parallelism_tradeoffs():
    bf16 = P.LoRALLMPredictor(P.synthesize_profile("llama-3.1-70b", quantized=False))
    nf4 = P.LoRALLMPredictor(P.synthesize_profile("llama-3.1-70b", quantized=True))
    one = P.SimulationConfiguration(dp=1, tp=1, pp=1, microbatch_tokens=16384, microbatches_per_step=2)
    assert not bf16.estimate(one).fits          # 140 GB of bf16 weights + activations > 180 GB
    r = nf4.estimate(one)
    assert r.fits and 1000 < r.tokens_per_s < 6000
    tp4pp2 = P.SimulationConfiguration(dp=1, tp=4, pp=2, microbatch_tokens=16384, microbatches_per_step=8)
    r2 = nf4.estimate(tp4pp2)
    assert r2.fits and r2.bubble_fraction == pytest.approx(1 / 9)
    dp8 = P.SimulationConfiguration(dp=8, microbatch_tokens=16384, microbatches_per_step=2)
    assert nf4.estimate(dp8).tokens_per_s > 6 * r.tokens_per_s
    best = P.best_configurations(nf4, 8, top=3)
    assert best and all(b[2].fits for b in best) and best[0][0] >= best[-1][0]


def test_b200_profiles_reproduce_measured_throughput():
    """The shipped B200 profiles (calibrated on measured layer times) predict the measured
    single-GPU and pipeline runs to within 15 %."""
    p8 = P.LoRALLMPredictor(P.load_b200_profile("llama-3.1-8b"))
    one = P.SimulationConfiguration(microbatch_tokens=16384, microbatches_per_step=3, recompute_layers=0,
                                    num_adapters=1)
    assert p8.estimate(one).tokens_per_s == pytest.approx(27731, rel=0.15)      # measured: cli.train, 1 GPU
    pp4dp2 = P.SimulationConfiguration(dp=2, pp=4, microbatch_tokens=16384, microbatches_per_step=15,
                                       recompute_layers=0)
    assert p8.estimate(pp4dp2).tokens_per_s == pytest.approx(144030, rel=0.15)  # measured: 8 GPUs
    prof = P.load_b200_profile("llama-3.1-70b")
    assert prof.layer_fwd_bwd(4096) == pytest.approx(15.30) and prof.layer_fwd_bwd(8192) == pytest.approx(29.96)
    # calibration keeps measured points exact and scales the rest of the grid
    synth = P.synthesize_profile("qwen2.5-32b")
    cal = P.calibrate_profile(synth, layer_fwd_bwd_ms={4096: 9.06}, head_fwd_bwd_ms={4096: 11.26})
    assert cal.layer_fwd_bwd(4096) == pytest.approx(9.06) and cal.head_fwd_bwd(4096) == pytest.approx(11.26)
    assert cal.layer_fwd_bwd(8192) / cal.layer_fwd_bwd(4096) == pytest.approx(
        synth.layer_fwd_bwd(8192) / synth.layer_fwd_bwd(4096))
