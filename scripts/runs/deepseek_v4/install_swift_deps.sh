#!/bin/bash
set -e
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../deps/swift_deps.sh"
rm -rf ~/.cache/huggingface/modules/transformers_modules/
