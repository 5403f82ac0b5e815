#!/usr/bin/env bash
# Every experiment of the evaluation, then the result table and the figures; counterpart of the
# reference's scripts/run_all.sh.  Each step can be run on its own.
set -uo pipefail
cd "$(dirname "$0")/.."
benchmarks/kernel_perf/1_kernel_perf.sh
for s in benchmarks/main/[123]_[1-5]_*.sh; do "$s" || echo "FAILED: $s"; done
benchmarks/scaling/70b_dp_scaling.sh
python -m lorafusion_b200.cli.parse_results outputs/main/*/results.csv --baseline-schedule mlora --plot outputs/figs \
  --csv outputs/main_results.csv
python -m lorafusion_b200.cli.figures kernel-perf --results outputs/kernel_perf/lora_kernels.jsonl --out outputs/figs
