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
  TR=(python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1)
  "${TR[@]}" --master-port 29531 bench.py --gpus "$N" --steps 3 --warmup 3
  if (( N % 2 == 0 )); then      # parameter sharding x tensor parallelism arm
    "${TR[@]}" --master-port 29532 bench.py --gpus "$N" --steps 2 --warmup 3 --skip-e2e --parallelism fsdp_tp2
  fi
  # peer-memory kernels against their NCCL twins and the link roofline; context-sharded attention transports
  NCCL_NVLS_ENABLE=0 "${TR[@]}" --master-port 29533 -m turbo_dllm_b200.benchmarks.comm_bench
  NCCL_NVLS_ENABLE=0 "${TR[@]}" --master-port 29534 -m turbo_dllm_b200.benchmarks.csbp_attention_bench --seq 32768
else
  python -m turbo_dllm_b200.benchmarks.attention_bench --seq 8192 --views 2 --bwd-modes fused
  python bench.py --gpus 1 --steps 3 --warmup 3
fi
