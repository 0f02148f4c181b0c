#!/bin/bash
# Qwen3-30B-A3B shape, EP 8, the engine's own loop
#   bash scripts/runs/qwen3/moe_30b_a3b_ep8.sh                       # synthetic tokens, random weights of the named shape
#   MODEL=/ckpt/hf DATA=train.jsonl bash scripts/runs/qwen3/moe_30b_a3b_ep8.sh
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common.sh"

OUTPUT_DIR=${OUTPUT_DIR:-/tmp/ttb200-own/moe_30b_a3b}
SEQ_LEN=${SEQ_LEN:-4096}
TT_CONFIG=${TT_CONFIG:-${RUNS_DIR}/qwen3/moe_30b_a3b_ep8.yaml}
start_log "$OUTPUT_DIR"
if [ -n "${MODEL:-}" ]; then SRC="--model $MODEL"; else SRC="--model_config ${RUNS_DIR}/qwen3/moe_30b_a3b.json"; fi
if [ -n "${DATA:-}" ]; then DATA_ARGS="--data $DATA"; else DATA_ARGS="--synthetic"; fi

torchrun $DISTRIBUTED_ARGS "${RUNS_DIR}/run_sft.py" --tt_config "${TT_CONFIG}" $SRC $DATA_ARGS \
    --seq_len "${SEQ_LEN}" --max_steps ${MAX_STEPS:-100} --lr ${LR:-1e-5} --logging_steps 10 --output_dir "$OUTPUT_DIR" \
    2>&1 | tee -a "$LOG_FILE"
