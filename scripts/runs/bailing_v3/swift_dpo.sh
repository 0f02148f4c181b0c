#!/bin/bash
# Ling / Bailing MoE V3 DPO on long pairs (ms-swift)
#   bash scripts/runs/bailing_v3/install_swift_deps.sh && bash scripts/runs/bailing_v3/swift_dpo.sh
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common.sh"

MODEL=${MODEL:-/models/Ling-flash-3.0-bf16}
OUTPUT_DIR=${OUTPUT_DIR:-/tmp/ttb200-swift-dpo/$(basename "$MODEL")}
SEQ_LEN=${SEQ_LEN:-65536}
DATASET=${DATASET:-AI-ModelScope/alpaca-gpt4-data-en}
TT_CONFIG=${TT_CONFIG:-${RUNS_DIR}/bailing_v3/dpo.yaml}
start_log "$OUTPUT_DIR"

torchrun $DISTRIBUTED_ARGS "${RUNS_DIR}/run_swift.py" dpo \
    --tt_config "${TT_CONFIG}" \
    --model "$MODEL" --dataset "$DATASET" --max_length "${SEQ_LEN}" --packing true --padding_free true \
    --train_type ${TRAIN_TYPE:-full} --torch_dtype bfloat16 --attn_impl flash_attn \
    --per_device_train_batch_size 1 --gradient_accumulation_steps ${GA:-1} --num_train_epochs ${EPOCHS:-1} \
    --learning_rate ${LR:-1e-5} --lr_scheduler_type cosine --warmup_ratio 0.0 --seed 42 \
    --logging_steps 1 --report_to tensorboard --eval_strategy no --save_steps ${SAVE_STEPS:-500} --save_total_limit 1 \
    --dataset_num_proc 16 --output_dir "$OUTPUT_DIR" --rlhf_type dpo --beta 0.1 \
    2>&1 | tee -a "$LOG_FILE"
