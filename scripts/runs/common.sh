#!/bin/bash
# Shared preamble of the run recipes: one node with 8 B200 GPUs by default, one process per GPU.
# Sourced by the per-model launchers; every value can be overridden from the environment.
set -o pipefail
set -eu

RUNS_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REPO_ROOT="$(cd "${RUNS_DIR}/../.." && pwd)"
export PYTHONPATH="${REPO_ROOT}:${PYTHONPATH:-}"

export NNODES=${NNODES:-1}
export GPUS_PER_NODE=${GPUS_PER_NODE:-8}
export NODE_RANK=${NODE_RANK:-0}
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29511}

# NVLink domain: peer-memory kernels carry the expert-parallel, sequence-parallel and FSDP traffic; NCCL is the control plane.
export TORCHTURBO_P2P_WAIT_MS=${TORCHTURBO_P2P_WAIT_MS:-5000}
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}
export TOKENIZERS_PARALLELISM=false
export WANDB_DISABLED=${WANDB_DISABLED:-True}
export TRANSFORMERS_VERBOSITY=${TRANSFORMERS_VERBOSITY:-error}

# build the sm_100a library once per checkout (no-op when the sources did not change)
python -c "from torchturbo_b200.csrc.build import build; build()" >/dev/null

DISTRIBUTED_ARGS="--nproc-per-node ${GPUS_PER_NODE} --nnodes ${NNODES} --node-rank ${NODE_RANK} --master-addr ${MASTER_ADDR} --master-port ${MASTER_PORT}"

start_log() {   # start_log <output dir>  -> sets LOG_FILE
    mkdir -p "$1"
    LOG_FILE="$1/node${NODE_RANK}-$(date +%Y%m%d-%H%M%S).log"
    echo "output: $1" > "${LOG_FILE}"
}
