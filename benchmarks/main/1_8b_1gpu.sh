#!/usr/bin/env bash
# Llama-3.1-8B on one GPU: one adapter, then four adapters sharing microbatches (solver and the
# mLoRA-style schedule).  Mirrors the reference's scripts/main/1_*_8b_1h100_*.sh family.
set -euo pipefail
cd "$(dirname "$0")/../.."
NGPU=1 MODEL=llama-3.1-8b ADAPTERS=1 GBS=64 DATASETS=medium benchmarks/run_single.sh
NGPU=1 MODEL=llama-3.1-8b ADAPTERS=4 RANKS="16 16 32 64" GBS="32 32 32 32" benchmarks/run_single.sh
NGPU=1 MODEL=llama-3.1-8b ADAPTERS=4 RANKS="16 16 32 64" GBS="32 32 32 32" SCHEDULE=mlora benchmarks/run_single.sh
