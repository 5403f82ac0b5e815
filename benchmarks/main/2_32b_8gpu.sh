#!/usr/bin/env bash
# Qwen2.5-32B, four adapters, TP2 x PP4 on eight GPUs (fused all-gather->GEMM / GEMM->reduce-scatter).
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=8 MODEL=qwen2.5-32b PP=4 TP=2 ADAPTERS=4 RANKS=16 GBS="32 32 32 32" benchmarks/run_single.sh
NGPU=8 MODEL=qwen2.5-32b PP=4 TP=2 ADAPTERS=4 RANKS=16 GBS="32 32 32 32" SCHEDULE=mlora benchmarks/run_single.sh
