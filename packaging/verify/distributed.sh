#!/usr/bin/env bash
# Multi-rank tier. Without GPUs: gloo ranks on the CPU (host-side logic of every parallel mode).
# With GPUs (the caller provides at least two): the NCCL / peer-memory tests as well.
set -euo pipefail
cd "$(cd "$(dirname "$0")/../.." && pwd)"
python -m pytest tests -x -q -m "distributed and not gpu"
if python -c "import torch, sys; sys.exit(0 if torch.cuda.device_count() >= 2 else 1)"; then
  NCCL_NVLS_ENABLE="${NCCL_NVLS_ENABLE:-0}" python -m pytest tests/test_gpu_multi.py -x -q -m gpu
fi
