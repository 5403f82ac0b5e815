#!/usr/bin/env bash
# Weak scaling of the flagship step (70B NF4, four adapters, data parallel with the fused
# reduce-scatter + AdamW + all-gather kernel) on 1, 2, 4 and 8 GPUs of one node.
set -euo pipefail
cd "$(dirname "$0")/../.."
for N in 1 2 4 8; do
  if [ "$N" -eq 1 ]; then python bench.py --gpus 1 --steps 3 --warmup 3
  else python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 \
         --master-port $((29500 + N)) bench.py --gpus "$N" --steps 3 --warmup 3; fi
done
