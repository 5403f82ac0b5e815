#!/usr/bin/env bash
# Kernel- and layer-level benchmarks (reference: scripts/kernel_perf/1_kernel_perf.sh and
# scripts/layer_perf/*.sh).
set -euo pipefail
cd "$(dirname "$0")/../.."
mkdir -p outputs/kernel_perf
python -m lorafusion_b200.cli.bench_kernels --shapes 4096x4096 5120x5120 8192x8192 --tokens 4096 8192 16384 \
  --reference-triton --csv outputs/kernel_perf/lora_kernels.csv | tee outputs/kernel_perf/lora_kernels.jsonl
python -m lorafusion_b200.cli.bench_kernels --nf4-compare --shapes 8192x8192 8192x28672 --tokens 256 1024 4096 16384
python -m lorafusion_b200.cli.bench_block_ops --model llama-3.1-70b --tokens 16384 --seq-len 4096
for M in llama-3.1-8b qwen2.5-32b llama-3.1-70b; do
  python -m lorafusion_b200.cli.bench_layer --model "$M" --seq-len 1024 --batch-sizes 4 8 16
done
