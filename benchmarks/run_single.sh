#!/usr/bin/env bash
# One training benchmark run: maps a few environment variables to the flags of
# `python -m lorafusion_b200.cli.train`, launches one process per GPU and appends the result
# line to $OUT/results.csv (written by the CLI itself).  Stands in for the reference's
# benchmarks_paper/scripts/run_single.sh (flag mapping, OOM detection by log grep, results.csv).
#
#   NGPU=8 MODEL=llama-3.1-70b QUANT=true PP=2 TP=4 ADAPTERS=4 RANKS="16" GBS="32 32 32 32" \
#   CAPACITY=16384 STEPS=3 benchmarks/run_single.sh
set -euo pipefail
NGPU=${NGPU:-1}; MODEL=${MODEL:-llama-3.1-8b}; QUANT=${QUANT:-false}
PP=${PP:-1}; TP=${TP:-1}; ADAPTERS=${ADAPTERS:-1}; RANKS=${RANKS:-16}; GBS=${GBS:-32}
CAPACITY=${CAPACITY:-16384}; STEPS=${STEPS:-3}; SCHEDULE=${SCHEDULE:-solver}
DATASETS=${DATASETS:-"short medium long xlong"}; OUT=${OUT:-outputs/${MODEL}_n${NGPU}_pp${PP}_tp${TP}_${SCHEDULE}}
PORT=${PORT:-$((29500 + RANDOM % 400))}
mkdir -p "$OUT"
ARGS=(--model_name_or_path "$MODEL" --load_in_4bit "$QUANT" --pipeline_parallel_size "$PP"
      --tensor_parallel_size "$TP" --multi_lora_max_microbatch_tokens "$CAPACITY"
      --multi_lora_global_batch_sizes "$GBS" --max_steps "$STEPS" --gradient_checkpointing_layers 1
      --adapter_to_dataset "$DATASETS" --output_dir "$OUT")
if [ "$ADAPTERS" -gt 1 ]; then
  ARGS+=(--use_multi_lora true --num_multi_loras "$ADAPTERS" --multi_lora_r "$RANKS")
else
  ARGS+=(--lora_r "${RANKS%% *}")
fi
[ "$SCHEDULE" = "mlora" ] && ARGS+=(--benchmark_baseline_mlora_schedule true)
[ -n "${SCHEDULE_PATH:-}" ] && ARGS+=(--multi_lora_dataset_schedule_path "$SCHEDULE_PATH")
if [ "$NGPU" -gt 1 ]; then
  LAUNCH=(python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port "$PORT" -m lorafusion_b200.cli.train)
else
  LAUNCH=(python -m lorafusion_b200.cli.train)
fi
set +e
"${LAUNCH[@]}" "${ARGS[@]}" > "$OUT/run.log" 2>&1
RC=$?
set -e
if grep -q "out of memory" "$OUT/run.log"; then echo "OOM: $OUT" | tee -a "$OUT/status.txt"; exit 3; fi
if [ $RC -ne 0 ]; then echo "FAILED rc=$RC: see $OUT/run.log"; tail -5 "$OUT/run.log"; exit $RC; fi
grep '"throughput_tokens_per_s"' "$OUT/run.log" | tail -1
