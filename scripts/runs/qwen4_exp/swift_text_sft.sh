#!/bin/bash
# Qwen4-exp text SFT (ms-swift): sparse attention, host-resident n-gram tables
#   bash scripts/runs/qwen4_exp/install_swift_deps.sh && bash scripts/runs/qwen4_exp/swift_text_sft.sh
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common.sh"

MODEL=${MODEL:-/models/Qwen4-exp}
OUTPUT_DIR=${OUTPUT_DIR:-/tmp/ttb200-swift-sft/$(basename "$MODEL")}
SEQ_LEN=${SEQ_LEN:-32768}
DATASET=${DATASET:-AI-ModelScope/alpaca-gpt4-data-en}
TT_CONFIG=${TT_CONFIG:-${RUNS_DIR}/qwen4_exp/swift_text_sft.yaml}
start_log "$OUTPUT_DIR"

torchrun $DISTRIBUTED_ARGS "${RUNS_DIR}/run_swift.py" sft \
    --tt_config "${TT_CONFIG}" \
    --model "$MODEL" --dataset "$DATASET" --max_length "${SEQ_LEN}" --packing true --padding_free true \
    --train_type ${TRAIN_TYPE:-full} --torch_dtype bfloat16 --attn_impl flash_attn \
    --per_device_train_batch_size 1 --gradient_accumulation_steps ${GA:-1} --num_train_epochs ${EPOCHS:-1} \
    --learning_rate ${LR:-1e-5} --lr_scheduler_type cosine --warmup_ratio 0.0 --seed 42 \
    --logging_steps 1 --report_to tensorboard --eval_strategy no --save_steps ${SAVE_STEPS:-500} --save_total_limit 1 \
    --dataset_num_proc 16 --output_dir "$OUTPUT_DIR"  \
    2>&1 | tee -a "$LOG_FILE"
