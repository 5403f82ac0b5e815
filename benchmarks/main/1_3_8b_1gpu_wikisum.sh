#!/usr/bin/env bash
# llama-3.1-8b, four adapters on the "wikisum" length profile(s), solver schedule and mLoRA-style
# schedule; counterpart of the reference's scripts/main/1_3_8b_1h100_wikisum.sh.
set -euo pipefail
cd "$(dirname "$0")/../.."
for SCHEDULE in solver mlora; do
  NGPU=1 MODEL=llama-3.1-8b QUANT=false PP=1 TP=1 ADAPTERS=4 RANKS=16 GBS="8 8 8 8" DATASETS="wikisum wikisum wikisum wikisum" \
    SCHEDULE=$SCHEDULE OUT=outputs/main/8b_wikisum_$SCHEDULE benchmarks/run_single.sh
done
