#!/usr/bin/env bash
# GPU smoke: release gates, the kernel library matches its manifest, one smoke recipe through the launcher.
#   packaging/verify/gpu_smoke.sh [RECIPE]        (default: cuda-fast-dllm-v2)
set -euo pipefail
cd "$(cd "$(dirname "$0")/../.." && pwd)"
RECIPE="${1:-cuda-fast-dllm-v2}"
python -m turbo_dllm_b200.profiling.release_gates > /dev/null
python -m turbo_dllm_b200.cli.main doctor
python -m turbo_dllm_b200.cli.main launch --recipe "$RECIPE" --nproc-per-node 1 --master-addr 127.0.0.1
