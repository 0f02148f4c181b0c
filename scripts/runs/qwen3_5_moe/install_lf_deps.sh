#!/bin/bash
set -e
source "$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)/../deps/lf_deps.sh"
# remote-code modules cached for another transformers version confuse `trust_remote_code` loads
rm -rf ~/.cache/huggingface/modules/transformers_modules/
