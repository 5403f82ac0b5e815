#!/usr/bin/env bash
# Nsight Compute capture of the fused LoRA linear kernels on a small case, summarised as a
# markdown table (reference: scripts/kernel_perf/2_kernel_ncu_profile.sh + summarize_kernel_ncu_profile.py).
# The plain command runs first; ncu only starts if it exited 0.  Clocks are left alone.
set -euo pipefail
cd "$(dirname "$0")/../.."
mkdir -p outputs/ncu
CMD=(python -m lorafusion_b200.cli.bench_kernels --shapes 8192x8192 --tokens 8192 --number 2 --profile-only fused_fwd_bwd)
"${CMD[@]}" > outputs/ncu/plain.log 2>&1 &&
ncu --set full --clock-control none -k regex:umma_gemm -c 12 -f -o outputs/ncu/fused_lora_linear "${CMD[@]}" > outputs/ncu/ncu.log 2>&1
ncu -i outputs/ncu/fused_lora_linear.ncu-rep --page raw --csv > outputs/ncu/fused_lora_linear.csv
python -m lorafusion_b200.cli.summarize_ncu outputs/ncu/fused_lora_linear.csv | tee outputs/ncu/fused_lora_linear.md
