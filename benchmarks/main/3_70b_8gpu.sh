#!/usr/bin/env bash
# Llama-3.1-70B with an NF4 base, four adapters, TP4 x PP2 on eight GPUs; counterpart of the
# reference's scripts/main/3_4_70b_4h100_mix.sh (PP4 on 4 x H100).
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=8 MODEL=llama-3.1-70b QUANT=true PP=2 TP=4 ADAPTERS=4 RANKS=16 GBS="32 32 32 32" benchmarks/run_single.sh
NGPU=8 MODEL=llama-3.1-70b QUANT=true PP=2 TP=4 ADAPTERS=4 RANKS=16 GBS="32 32 32 32" SCHEDULE=mlora benchmarks/run_single.sh
