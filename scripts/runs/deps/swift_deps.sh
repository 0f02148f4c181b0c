#!/bin/bash
# ms-swift 4.x stack the `msswift` adapter is gated for.
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/platform.sh"
pip install "transformers>=5.5" safetensors==0.7.0 "peft>=0.18,<0.19" "datasets>=4.0" "accelerate>=1.11,<1.12" "trl>=0.29,<0.30" \
    binpacking tensorboard psutil pyyaml matplotlib
pip install "ms_swift>=4.4,<5"
