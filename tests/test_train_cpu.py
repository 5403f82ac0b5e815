"""CPU tests of the training front end: argument groups, data providers, schedule-driven
microbatch specs."""

import pytest

from lorafusion_b200.models.config import AdapterSpec
from lorafusion_b200.solver import schedule as S
from lorafusion_b200.train.args import (MockDataArguments, ModelArguments, TrainingArguments,
                                        parse_args_into_dataclasses, parse_list)
from lorafusion_b200.train.data import MockDataset, NAMED_DISTRIBUTIONS
from lorafusion_b200.train.provider import DataProvider, MockMultiLoRADataProvider


def test_argument_groups_parse_reference_style_flags():
    m, t, d = parse_args_into_dataclasses([
        "--model_name_or_path", "llama-3.1-70b", "--load_in_4bit", "true", "--use_multi_lora", "true",
        "--num_multi_loras", "4", "--multi_lora_r", "16 16 32 64", "--multi_lora_alpha", "32",
        "--multi_lora_dropout_p", "0.1,0.1,0.0,0.05", "--pipeline_parallel_size", "2",
        "--tensor_parallel_size", "4", "--multi_lora_global_batch_sizes", "8 8 16 16",
        "--apply_fused_lora", "true", "--liger_kernel_level", "all", "--dataset_name", "mix"])
    assert isinstance(m, ModelArguments) and isinstance(t, TrainingArguments) and isinstance(d, MockDataArguments)
    specs = m.adapter_specs()
    assert [s.r for s in specs] == [16, 16, 32, 64] and [s.name for s in specs] == [f"lora_{i}" for i in range(4)]
    assert [s.dropout for s in specs] == [0.1, 0.1, 0.0, 0.05] and all(s.lora_alpha == 32.0 for s in specs)
    assert m.load_in_4bit is True and t.pipeline_parallel_size == 2 and t.tensor_parallel_size == 4
    assert parse_list(t.multi_lora_global_batch_sizes, int) == [8, 8, 16, 16]
    with pytest.raises(SystemExit):
        parse_args_into_dataclasses(["--no_such_flag", "1"])
    with pytest.raises(ValueError):
        ModelArguments(use_multi_lora=True, num_multi_loras=3, multi_lora_r="16 32").adapter_specs()
    # single adapter
    (single,) = ModelArguments(lora_r=8, lora_alpha=16, lora_dropout=0.0).adapter_specs()
    assert single.r == 8 and single.scaling == 2.0


def test_global_batch_invariant():
    t = TrainingArguments(per_device_train_batch_size=2, global_batch_size=32)
    t.resolve_batch(dp_size=4)
    assert t.gradient_accumulation_steps == 4
    t2 = TrainingArguments(per_device_train_batch_size=2, gradient_accumulation_steps=3)
    t2.resolve_batch(dp_size=2)
    assert t2.global_batch_size == 12
    with pytest.raises(ValueError):
        TrainingArguments(per_device_train_batch_size=3, global_batch_size=32).resolve_batch(dp_size=4)
    assert TrainingArguments(gradient_checkpointing=False).recompute_mode() is False
    assert TrainingArguments(gradient_checkpointing_layers=4).recompute_mode() == "auto"


def test_multi_lora_provider_covers_every_sample_once():
    adapters = [AdapterSpec(f"lora_{i}", r=16) for i in range(3)]
    prov = MockMultiLoRADataProvider.from_named_distributions(
        adapters, ["short", "medium", "xlong"], [8, 8, 4], num_samples=40, seed=1, max_len=4096, capacity=8192,
        num_pipeline_stages=2, vocab_size=1000, num_global_batches=3, use_exact=False, num_workers=1)
    mbs = prov.microbatches()
    assert len(mbs) == len(prov) and len(mbs) > 3
    seen = {}
    for mb in mbs:
        if mb.is_empty:
            continue
        assert mb.spec.total_tokens <= 8192
        for (a, g, k), ln in mb.info.data_samples.items():
            assert (a, g, k) not in seen
            seen[(a, g, k)] = ln
    expected = {(a, g, k): ln for a, batches in enumerate(prov.data) for g, b in enumerate(batches)
                for k, ln in enumerate(b)}
    assert seen == expected
    assert S.bubble_lemma_violations(prov.flat, 2) == []
    stats = prov.statistics()
    assert stats["num_microbatches"] + stats["num_noops"] == len(mbs)
    # padded totals follow the requested multiple (needed by tensor parallelism)
    prov4 = MockMultiLoRADataProvider(adapters, prov.datasets, [8, 8, 4], capacity=8192, num_pipeline_stages=2,
                                      vocab_size=1000, num_global_batches=2, use_exact=False, num_workers=1,
                                      total_multiple=512)
    assert all(mb.spec.padded_total_tokens % 512 == 0 for mb in prov4.microbatches() if not mb.is_empty)


def test_single_adapter_provider_packs_up_to_capacity_and_strides_over_dp_ranks():
    ds = MockDataset.from_distribution(NAMED_DISTRIBUTIONS["medium"], 64, seed=0)
    provs = [DataProvider(AdapterSpec("default", r=16), ds, capacity=4096, vocab_size=100, dp_rank=r, dp_size=2)
             for r in range(2)]
    specs = [p.next_spec() for p in provs]
    for s in specs:
        assert 0 < s.total_tokens <= 4096 and s.padded_total_tokens <= 4096 + 128
    lens0 = [ln for _, lens in specs[0].segments for ln in lens]
    lens1 = [ln for _, lens in specs[1].segments for ln in lens]
    assert lens0 == ds.lengths[0:2 * len(lens0):2] and lens1 == ds.lengths[1:2 * len(lens1):2]
