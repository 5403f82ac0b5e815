#!/usr/bin/env bash
# llama-3.1-70b, four adapters on the "xsum" length profile(s), solver schedule and mLoRA-style
# schedule; counterpart of the reference's scripts/main/3_1_70b_4h100_xsum.sh.
set -euo pipefail
cd "$(dirname "$0")/../.."
for SCHEDULE in solver mlora; do
  NGPU=8 MODEL=llama-3.1-70b QUANT=true PP=2 TP=4 ADAPTERS=4 RANKS=16 GBS="16 16 16 16" DATASETS="xsum xsum xsum xsum" \
    SCHEDULE=$SCHEDULE OUT=outputs/main/70b_xsum_$SCHEDULE benchmarks/run_single.sh
done
