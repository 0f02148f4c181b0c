#!/bin/bash
# LlamaFactory 0.9.x stack the `llamafactory_v0` adapter is gated for (registry/adapter.py checks the version).
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/platform.sh"
pip install "transformers>=5.5,<5.6" safetensors==0.7.0 "peft>=0.18,<0.19" "datasets>=4.0,<4.1" "accelerate>=1.11,<1.12" \
    "trl>=0.24,<0.25" tensorboard psutil pyyaml matplotlib
pip install "llamafactory>=0.9.4,<0.10"
