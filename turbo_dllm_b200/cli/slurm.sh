#!/usr/bin/env bash
# Thin wrapper for Slurm allocations: run once per node (srun --ntasks-per-node=1 ./slurm.sh --config train.yaml).
# Node count, node rank and the rendezvous host come from Slurm's environment.
# Counterpart of the reference's scripts/launch/slurm.sh.
set -euo pipefail
head_node="$(scontrol show hostnames "${SLURM_JOB_NODELIST}" | head -n 1)"
exec python -m turbo_dllm_b200.cli.main launch --nnodes "${SLURM_JOB_NUM_NODES:-1}" \
  --node-rank "${SLURM_NODEID:-0}" --nproc-per-node "${NPROC:-8}" \
  --master-addr "${head_node}" --master-port "${MASTER_PORT:-29500}" "$@"
