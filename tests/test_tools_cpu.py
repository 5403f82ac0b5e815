"""CPU tests of the result tooling: SVG charts, dataset-distribution generator, result parser and
the Nsight Compute summariser."""

import csv
import json
import xml.dom.minidom as minidom

from lorafusion_b200.cli import gen_sample_distribution, parse_results, summarize_ncu
from lorafusion_b200.train.data import MockDataset
from lorafusion_b200.utils.plotting import GroupedBarChart, MultiLinePlot, PipelineGantt, StackedBarChart


def test_charts_are_valid_svg(tmp_path):
    charts = [
        GroupedBarChart(["8B", "70B"], ["base", "ours"], [[1.0, 2.0], [1.5, 3.9]], title="a<b", normalize_to="base"),
        StackedBarChart(["x", "y"], ["gemm", "attn"], [[3, 4], [1, 2]], ylabel="ms"),
        MultiLinePlot(["s1", "s2"], [[1, 2, 4, 8]] * 2, [[1, 2, 4, 7.9], [1, 1.8, 3.1, 5]], logx=True),
        PipelineGantt([[(0, 1), (1, 2)], [(1, 2), (2, 3)]], [[(4, 6), (6, 8)], [(3, 4), (4, 6)]], title="1F1B"),
    ]
    for i, c in enumerate(charts):
        path = c.save(tmp_path / f"c{i}.svg")
        doc = minidom.parse(str(path))
        assert doc.documentElement.tagName == "svg" and len(doc.getElementsByTagName("rect")) >= 1
    # normalisation: the baseline series becomes 1.0 everywhere
    assert charts[0].values[0] == [1.0, 1.0] and abs(charts[0].values[1][1] - 1.95) < 1e-9


def test_gen_sample_distribution_layout(tmp_path, capsys):
    out = tmp_path / "d.json"
    gen_sample_distribution.main(["--out", str(out), "--datasets", "xsum", "wikisum", "mix", "het", "--seeds", "0", "3",
                                  "--permutations", "2", "--num-samples", "120", "--plot"])
    data = json.loads(out.read_text())
    assert set(data) == {"xsum", "wikisum", "mix", "het"} and set(data["mix"]) == {"seed_0", "seed_3"}
    p1, p2 = data["xsum"]["seed_0"]["permutation_1"], data["xsum"]["seed_0"]["permutation_2"]
    assert len(p1) == 120 and sorted(p1) == sorted(p2) and p1 != p2 and max(p1) <= 4096
    # readable by the dataset loader
    ds = MockDataset.from_distribution_file(out, "wikisum", seed=3, permutation=2)
    assert len(ds) == 120 and out.with_suffix(".svg").exists()
    rows = [json.loads(ln) for ln in capsys.readouterr().out.strip().splitlines()]
    assert {r["dataset"] for r in rows} == {"xsum", "wikisum", "mix", "het"}


def test_parse_results_speedups(tmp_path, capsys):
    fields = ["model", "layout", "world", "adapters", "capacity", "microbatches", "tokens", "time_ms",
              "throughput_tokens_per_s", "throughput_per_gpu", "peak_memory_gib", "bubble_ratio",
              "optimizer_steps", "quantized", "schedule"]
    path = tmp_path / "results.csv"
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=fields)
        w.writeheader()
        for sched, tps in (("solver", 1500.0), ("mlora", 1000.0), ("solver", 1400.0)):
            w.writerow(dict(model="m", layout="dp1pp4tp1", world=4, adapters=4, capacity=16384, microbatches=10,
                            tokens=1e5, time_ms=1.0, throughput_tokens_per_s=tps, throughput_per_gpu=tps / 4,
                            peak_memory_gib=10.0, bubble_ratio="", optimizer_steps="{}", quantized=False,
                            schedule=sched))
    sp = parse_results.main([str(path), "--plot", str(tmp_path / "figs")])
    assert len(sp) == 1 and abs(sp[0]["speedup"] - 1.5) < 1e-9
    assert (tmp_path / "figs" / "end_to_end.svg").exists() and (tmp_path / "figs" / "scaling.svg").exists()


def test_summarize_ncu_tables(tmp_path):
    raw = tmp_path / "raw.csv"
    raw.write_text('"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum",'
                   '"sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active","launch__grid_size"\n'
                   '"","","us","Mbyte","%",""\n'
                   '"0","void lf::k<1, 2>(P)","761.3","1101.4","86.98","148"\n')
    text = summarize_ncu.main([str(raw)])
    assert "`lf::k<1, 2>`" in text and "86.98" in text and "761.3 us" in text
    launches = tmp_path / "l.csv"
    launches.write_text('==PROF== Connected\n"ID","Kernel Name","Metric Name","Metric Unit","Metric Value"\n'
                        '"0","a(int)","gpu__time_duration.sum","ns","3000000"\n'
                        '"1","b(int)","gpu__time_duration.sum","ns","1000000"\n'
                        '"2","a(int)","gpu__time_duration.sum","ns","1000000"\n')
    text = summarize_ncu.main([str(launches), "--launches"])
    assert "Total 5.0 ms over 3 launches" in text and "| `a` | 2 | 4.000 | 80.0 % |" in text


def test_tile_config_registry_round_trip(tmp_path, monkeypatch):
    """What the tuner writes is what the launchers read; unknown shapes fall back to defaults."""
    from lorafusion_b200.ops import tile_config as tc

    path = tmp_path / "table.json"
    tc.write_table({tc.entry_key("fwd", 16000, 8192, 28672): {"group_m": 16, "max_ctas": 132, "tflops": 1400.0}},
                   path, gpu="test-gpu")
    monkeypatch.setenv("LORAFUSION_B200_TUNING", str(path))
    tc.reload()
    got = tc.get_kernel_config("fwd", 16384, 8192, 28672)          # same power-of-two bucket as 16000
    assert (got.group_m, got.max_ctas, got.source) == (16, 132, str(path))
    assert tc.get_kernel_config("fwd", 4096, 8192, 28672) == tc.DEFAULTS["fwd"]
    assert tc.get_kernel_config("dx", 16384, 8192, 28672).group_m == 8
    tc.write_table({tc.entry_key("dx", 16384, 28672, 8192): {"group_m": 4, "max_ctas": 0}}, path, gpu="test-gpu")
    assert tc.get_kernel_config("dx", 16384, 28672, 8192).group_m == 4
    assert tc.get_kernel_config("fwd", 16384, 8192, 28672).group_m == 16   # merged, not replaced
    monkeypatch.delenv("LORAFUSION_B200_TUNING")
    tc.reload()


def test_figure_drivers_draw_published_and_measured_data(tmp_path):
    import json

    from lorafusion_b200.cli import figures

    for name, n in (("end-to-end", 3), ("scaling", 1), ("kernel-dram", 1)):
        paths = figures.main([name, "--demo", "--out", str(tmp_path)])
        assert len(paths) == n and all(p.read_text().lstrip().startswith("<svg") for p in paths)
    (tmp_path / "scale.json").write_text(json.dumps({"scaling": {"values": {"1": 2800.0, "2": 5400.0, "8": 21000.0}}}))
    p, = figures.main(["scaling", "--results", str(tmp_path / "scale.json"), "--out", str(tmp_path)])
    assert "this framework" in p.read_text()
    rows = [{"shape": f"[{m}x4096x4096x16] FWD", "torch_lora_s": 3e-4 * m / 4096, "torch_linear_s": 2e-4 * m / 4096,
             "fused_lora_s": 2.5e-4 * m / 4096, "fused_multi_lora_4x_s": 2.6e-4 * m / 4096} for m in (4096, 8192)]
    (tmp_path / "k.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    p, = figures.main(["kernel-perf", "--results", str(tmp_path / "k.jsonl"), "--out", str(tmp_path)])
    assert "FusedLoRA" in p.read_text() and "Reference Triton" not in p.read_text()
    layer = [{"Mode": "FusedLoRA", "Model": "llama-3.1-8b", "BatchSize": b, "SeqLength": 1024, "NumAdapters": 1,
              "TimeMs": 5.0 * b, "ThroughputTokensPerSec": 1.0} for b in (4, 8)]
    (tmp_path / "l.jsonl").write_text("\n".join(json.dumps(r) for r in layer))
    p, = figures.main(["layer-perf", "--results", str(tmp_path / "l.jsonl"), "--out", str(tmp_path)])
    assert "llama-3.1-8b" in p.read_text()


def test_packed_dummy_inputs_and_verbose_allclose():
    """Helpers with the reference's names: packed varlen inputs (positions restart per sequence,
    padding forms one more sequence) and an allclose that reports instead of raising."""
    import torch

    from lorafusion_b200.utils import create_packed_dummy_inputs, verbose_allclose

    d = create_packed_dummy_inputs(32, [5, 3], multiple_of=16, device="cpu", return_labels=True,
                                   return_inputs_embeds=True, seed=1)
    assert d["cu_seq_lens_q"].tolist() == [0, 5, 8, 16] and d["cu_seq_lens_q"].dtype == torch.int32
    assert d["position_ids"][0].tolist() == [0, 1, 2, 3, 4, 0, 1, 2] + list(range(8))
    assert d["input_ids"].shape == (1, 16) and int(d["input_ids"].max()) < 10000
    assert d["inputs_embeds"].shape == (1, 16, 32) and d["labels"].shape == (1, 16)
    assert d["max_length_q"] == 8
    said = []
    assert verbose_allclose(torch.ones(4), torch.ones(4), print_fn=said.append) and not said
    assert not verbose_allclose(torch.ones(4), torch.tensor([1.0, 1.0, 2.0, 1.0]), msg="x", print_fn=said.append)
    assert "1/4 mismatched" in said[0]


def test_offload_slots_are_sized_exactly():
    """A host slot takes its size rounded to pages, not to a power of two: the 1.75 GiB gate|up
    output of a 16K-token 70B microbatch fits 49 times into 92 GB, not 43 times."""
    from lorafusion_b200.models.offload import host_slot_bytes

    per_gu = 16384 * 2 * 28672 * 2
    assert host_slot_bytes(per_gu) == per_gu            # already a multiple of 4096
    assert host_slot_bytes(per_gu + 1) == per_gu + 4096
    budget = int(0.45 * 205.8e9)
    assert budget // host_slot_bytes(per_gu) == 49
    assert budget // (1 << (per_gu - 1).bit_length()) == 43


def test_bench_reference_arm_prints_one_unavailable_line():
    """``bench.py --impl reference`` cannot run the reference on this image: it says so in one
    JSON line and exits 0, also when every rank of a multi-process launch calls it."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path

    bench = Path(__file__).resolve().parents[1] / "bench.py"
    for rank, expect_lines in ((0, 1), (1, 0)):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank))
        res = subprocess.run([sys.executable, str(bench), "--impl", "reference", "--gpus", "2", "--steps", "2",
                              "--warmup", "1"], capture_output=True, text=True, timeout=300, env=env)
        assert res.returncode == 0, res.stderr[-2000:]
        lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
        assert len(lines) == expect_lines
        if lines:
            rec = json.loads(lines[0])
            assert rec["impl"] == "reference" and "unavailable" in rec and "\n" not in rec["unavailable"]
