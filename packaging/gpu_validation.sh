#!/usr/bin/env bash
# Qualification of a built tree (or installed wheel) on a machine with B200 GPUs:
# release gates, the GPU test tier, the flagship smoke step and a short benchmark.
#   packaging/gpu_validation.sh [N_GPUS]
set -euo pipefail
N="${1:-1}"
ROOT="$(cd "$(dirname "$0")/.." && pwd)"
cd "$ROOT"
python -m turbo_dllm_b200.profiling.release_gates
python -m pytest tests -x -q -m gpu
python -c "import __graft_entry__ as g; g.smoke()"
if [[ "$N" -gt 1 ]]; then
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 --master-port 29531 \
      bench.py --gpus "$N" --steps 3 --warmup 3
else
  python bench.py --gpus 1 --steps 3 --warmup 3
fi
