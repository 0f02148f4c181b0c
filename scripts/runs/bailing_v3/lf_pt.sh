#!/bin/bash
# Ling / Bailing MoE V3 continued pre-training (LlamaFactory)
#   bash scripts/runs/bailing_v3/install_lf_deps.sh && bash scripts/runs/bailing_v3/lf_pt.sh
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../common.sh"

MODEL=${MODEL:-/models/Ling-flash-3.0-bf16}
OUTPUT_DIR=${OUTPUT_DIR:-/tmp/ttb200-lf-pt/$(basename "$MODEL")}
SEQ_LEN=${SEQ_LEN:-8192}
DATASET=${DATASET:-gsm8k}                       # registered in ${DATASET_DIR}/dataset_info.json
DATASET_DIR=${DATASET_DIR:-${REPO_ROOT}/dataset}
TT_CONFIG=${TT_CONFIG:-${RUNS_DIR}/bailing_v3/pt.yaml}
start_log "$OUTPUT_DIR"

torchrun $DISTRIBUTED_ARGS "${RUNS_DIR}/run_lf.py" \
    --tt_config "${TT_CONFIG}" \
    --stage pt --do_train --model_name_or_path "$MODEL" --template bailing_v3 --trust_remote_code \
    --dataset_dir "${DATASET_DIR}" --dataset "$DATASET" --cutoff_len "${SEQ_LEN}" --neat_packing --disable_shuffling \
    --preprocessing_num_workers 16 --overwrite_cache \
    --finetuning_type ${FINETUNING_TYPE:-full} --bf16 --flash_attn fa2 --gradient_checkpointing \
    --per_device_train_batch_size 1 --gradient_accumulation_steps ${GA:-1} --num_train_epochs ${EPOCHS:-1} \
    --learning_rate ${LR:-1.25e-5} --lr_scheduler_type cosine --warmup_ratio 0.0 --seed 42 \
    --logging_steps 1 --report_to tensorboard --plot_loss --eval_strategy no \
    --save_strategy steps --save_steps ${SAVE_STEPS:-500} --save_total_limit 1 \
    --output_dir "$OUTPUT_DIR" --overwrite_output_dir --ddp_timeout 1800  \
    2>&1 | tee -a "$LOG_FILE"
