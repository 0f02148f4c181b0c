#!/bin/bash
# CUDA 12.8+ wheels of PyTorch carry sm_100 code; the kernels of this package are built in-tree with nvcc >= 12.8.
pip install "torch>=2.10.0"
command -v nvcc >/dev/null || echo "warning: nvcc not on PATH; python -m torchturbo_b200.csrc.build needs CUDA >= 12.8" >&2
