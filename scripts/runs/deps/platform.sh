#!/bin/bash
# This package targets NVIDIA B200 (sm_100a) only: refuse to install anywhere else.
if ! nvidia-smi -L >/dev/null 2>&1; then
    echo "no NVIDIA GPU visible: torchturbo_b200 needs a Blackwell (sm_100a) device" >&2
    exit 1
fi
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/gpu.sh"
