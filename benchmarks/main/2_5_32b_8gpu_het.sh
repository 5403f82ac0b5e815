#!/usr/bin/env bash
# qwen2.5-32b, four adapters on the "het" length profile(s), solver schedule and mLoRA-style
# schedule; counterpart of the reference's scripts/main/2_5_32b_2h100_het.sh.
set -euo pipefail
cd "$(dirname "$0")/../.."
for SCHEDULE in solver mlora; do
  NGPU=8 MODEL=qwen2.5-32b QUANT=false PP=4 TP=2 ADAPTERS=4 RANKS=16 GBS="8 8 8 8" DATASETS="short medium long xlong" \
    SCHEDULE=$SCHEDULE OUT=outputs/main/32b_het_$SCHEDULE benchmarks/run_single.sh
done
